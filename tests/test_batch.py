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


def test_a_step_padded_to_a_bucket_keeps_its_rows_and_marks_the_rest_as_padding():
    from grout_b200.engine.batch import pack_step_padded
    rng = random.Random(9)
    for _ in range(200):
        n = rng.randint(0, 5)
        entries, want = [], []
        for i in range(n):
            q = rng.choice([1, 2, 5, 17])
            entries.append((rng.randint(0, 30), rng.choice([0, 3, 64]), [rng.randint(1, 999) for _ in range(q)]))
            want.append(sorted(rng.sample(range(q), rng.randint(0, min(q, 2)))))
        T = sum(len(e[2]) for e in entries)
        nt = T + rng.choice([0, 1, 13])
        ns = n + (1 if nt > T else 0) + rng.choice([0, 2])
        nw = sum(len(w) for w in want) + rng.choice([0, 3])
        if nt == 0:
            continue
        buf, meta = pack_step_padded(entries, want, nt, max(ns, 1), nw)
        plain, pmeta = pack_step(entries, want)
        off = meta["off"]

        def arr(name, m=meta, b=buf):
            o, cnt = m["off"][name]
            return b[o:o + cnt].tolist()

        for name in ("tokens", "token_seq", "token_pos"):          # the real rows are unchanged
            assert arr(name)[:T] == arr(name, pmeta, plain)
        assert arr("want_rows")[:meta["n_real_want"]] == arr("want_rows", pmeta, plain)
        assert arr("want_rows")[meta["n_real_want"]:] == [0] * (nw - meta["n_real_want"])
        cu, slots, kv = arr("cu_q"), arr("slots"), arr("kv_len")
        assert cu[:n + 1] == arr("cu_q", pmeta, plain) and cu[-1] == nt
        assert all(a <= b for a, b in zip(cu, cu[1:]))
        assert slots[:n] == [e[0] for e in entries] and all(s == -1 for s in slots[n:])
        if nt > T:                                                  # one sequence takes the rows left over
            assert cu[n + 1] == nt and arr("token_seq")[T:] == [n] * (nt - T)
            assert arr("token_pos")[T:] == list(range(nt - T)) and kv[n] == nt - T
        assert all(cu[i + 1] == cu[i] and kv[i] == 0 for i in range(n + (1 if nt > T else 0), len(slots)))
        assert len(meta["q_lens"]) == len(slots) and sum(meta["q_lens"]) == nt
    with pytest.raises(ValueError, match="do not fit"):
        pack_step_padded([(0, 0, [1, 2, 3])], [[0]], 2, 2, 1)
    with pytest.raises(ValueError, match="do not fit"):
        pack_step_padded([(0, 0, [1, 2, 3])], [[0]], 4, 1, 1)       # no sequence left for the padding rows
    with pytest.raises(ValueError, match="do not fit"):
        pack_step_padded([(0, 0, [1, 2, 3])], [[0, 1]], 4, 2, 1)


def test_buckets_of_the_captured_prompt_steps_and_of_the_lengths():
    from grout_b200.engine.graphs import (PROMPT_SEQS_MOST, PROMPT_TOKENS_MOST, length_bucket,
                                          prompt_bucket)
    from grout_b200.engine.batch import pack_step_padded
    for T in (1, 5, 16, 17, 64, 65, 1000, 1024):
        for n in (1, 2, 3, 31, 32, 33, 63, 64):
            if n > T:
                continue
            for w in (0, 1, n, T):
                key = prompt_bucket(T, n, w)
                need = n + (1 if T < max(16, 1 << (T - 1).bit_length()) else 0)
                if need > PROMPT_SEQS_MOST:
                    assert key is None
                    continue
                tb, sb, wb = key
                assert tb >= T and sb >= need and wb >= w and (w > 0) == (wb > 0)
                assert tb & (tb - 1) == 0 and sb & (sb - 1) == 0 and wb & (wb - 1) == 0
                # whatever the bucket, the step fits it
                q = [T // n + (1 if i < T % n else 0) for i in range(n)]
                entries = [(i, 0, [1] * q[i]) for i in range(n)]
                want = [[0] if i < w else [] for i in range(n)] if w <= n else [list(range(x)) for x in q]
                pack_step_padded(entries, want, tb, sb, wb)
    assert prompt_bucket(PROMPT_TOKENS_MOST + 1, 1, 1) is None
    assert [length_bucket(n, 4096) for n in (1, 512, 513, 2049, 4096)] == [512, 512, 1024, 4096, 4096]
    assert length_bucket(100, 320) == 320 and length_bucket(3000, 40960) == 4096


def test_the_blocks_a_kernel_sizes_its_grid_with():
    ctx = make_context([(0, 0, [1] * 70), (1, 5, [1] * 3), (2, 0, [1] * 64)], None, "cpu")
    assert ctx.q_blocks(64) == 2 + 1 + 1 and ctx.q_blocks(128) == 3
    ctx.q_lens = ()                          # a captured step: the most the rows can make
    assert ctx.q_blocks(64) == 137 // 64 + 3 >= 4
