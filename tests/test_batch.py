"""The packing of a step's batch into one int32 buffer, and the buckets of the captured
decode steps, on the host (no GPU)."""
import random

import pytest

from grout_b200.engine.batch import make_context, pack_step


def test_random_batches_are_packed_row_after_row():
    rng = random.Random(5)
    for _ in range(200):
        n = rng.randint(1, 7)
        entries, want = [], []
        for i in range(n):
            q = rng.choice([1, 1, 2, 5, 64, 65])
            start = rng.choice([0, 0, 3, 100])
            entries.append((rng.randint(0, 30), start, [rng.randint(0, 999) for _ in range(q)]))
            want.append(sorted(rng.sample(range(q), rng.randint(0, min(q, 3)))))
        pad = rng.choice([0, 0, 1, 3])
        buf, meta = pack_step(entries, want, pad)
        off = meta["off"]

        def arr(name):
            o, cnt = off[name]
            return buf[o:o + cnt].tolist()

        tokens, seq, pos, cu, rows = [], [], [], [0], []
        for i, (slot, start, toks) in enumerate(entries):
            rows += [len(tokens) + p for p in want[i]]
            tokens += toks
            seq += [i] * len(toks)
            pos += list(range(start, start + len(toks)))
            cu.append(len(tokens))
        for j in range(pad):                      # padding: one token, slot -1, position 0
            tokens.append(0), seq.append(n + j), pos.append(0), cu.append(len(tokens))
        assert arr("tokens") == tokens and arr("token_seq") == seq and arr("token_pos") == pos
        assert arr("cu_q") == cu and arr("want_rows") == rows
        assert arr("slots") == [e[0] for e in entries] + [-1] * pad
        assert arr("kv_len") == [e[1] + len(e[2]) for e in entries] + [1] * pad
        assert meta["n_tokens"] == len(tokens) and meta["n_seqs"] == n + pad and meta["n_want"] == len(rows)
        assert meta["decode"] == all(len(e[2]) == 1 for e in entries)
        assert meta["max_q_len"] == max(len(e[2]) for e in entries)
        assert meta["max_kv_len"] == max([e[1] + len(e[2]) for e in entries] + [1] * pad)
        # every array of the layout lies in the buffer, one after the other, none overlapping
        spans = sorted(off.values())
        assert spans[0][0] == 0 and all(a[0] + a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert spans[-1][0] + spans[-1][1] == buf.shape[0]


def test_wanted_places_are_checked():
    with pytest.raises(ValueError, match="outside"):
        pack_step([(0, 0, [1, 2, 3])], [[3]])
    with pytest.raises(ValueError, match="one list"):
        pack_step([(0, 0, [1]), (1, 0, [2])], [[0]])
    ctx = make_context([(4, 10, [7, 8])], None, "cpu")
    assert ctx.want_rows is None and ctx.n_want == 0 and ctx.kv_len.tolist() == [12]
    assert ctx.token_pos.tolist() == [10, 11] and ctx.slots.tolist() == [4]


def test_buckets_of_the_captured_decode_steps():
    from grout_b200.engine.graphs import bucket_for
    for largest in (1, 8, 64, 256):
        for n in range(1, 300):
            b = bucket_for(n, largest)
            if n > largest:
                assert not b
            else:
                assert b >= n and b & (b - 1) == 0 and b <= largest and (b == 1 or b // 2 < n)
