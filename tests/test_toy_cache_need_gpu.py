"""A third kind of cache need, and an embedding that adds learned positions,
defined here, in the test, and run by the library without a change to its files.

The toy mixer keeps one small latent vector per token (neither keys and values
nor a state of fixed size); its need, ``LatentSpec``, makes its own store, which
the cache holds beside the key/value store of the attention layer.  Both toy
parts read everything that varies from the step's device arrays, so they allow
their prompt steps to be captured; the test checks that the captured path ran.
The toy model is nobody's architecture; it only shows the interfaces."""
import os
from dataclasses import dataclass

import pytest
import torch

from conftest import random_tokens
from helpers import assert_close, run_batch, run_chunks, run_tail_decoded, run_whole
from plain import qwen3 as plain

TOY = dict(architectures=["ToyLatentForCausalLM"], model_type="toy_latent", vocab=113, width=56,
           inner=72, rank=12, heads=2, kv_heads=2, head_dim=32, eps=1e-5, theta=900.0,
           max_positions=192)


def _register():
    from grout_b200.config import register_architecture
    from grout_b200.config.base import ModelConfig
    from grout_b200.parts import (Embedding, LayerPlan, Mixer, ModelPlan, ParamSpec,
                                  PartSpec, ScheduleEntry, register_part)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab: int
        width: int
        inner: int
        rank: int
        heads: int
        kv_heads: int
        head_dim: int
        eps: float
        theta: float
        max_positions: int
        model_type: str = "toy_latent"
        architectures: tuple = ("ToyLatentForCausalLM",)

    # ---- the need and its store -------------------------------------------------
    @dataclass
    class LatentLayerView:
        latent: torch.Tensor          # [slots + 1, longest sequence, rank]; the last row is for padding

    class LatentStore:
        """One latent vector per token and layer.  Nothing is cleared when a slot
        is opened: a reader looks at positions up to its own only."""

        def __init__(self, spec, n_layers, sizes, device, allocate):
            self.spec, self.sizes = spec, sizes
            self.held = {}
            self.data = None
            if allocate:
                self.data = torch.zeros((n_layers, sizes.max_slots + 1, sizes.max_seq_len, spec.rank),
                                        dtype=torch.float32, device=device)

        def open(self, slot):
            assert slot not in self.held
            self.held[slot] = 0

        def reserve(self, slot, n_tokens):
            if n_tokens > self.sizes.max_seq_len:
                raise RuntimeError("sequence too long for the latent store")
            self.held[slot] = n_tokens

        def trim(self, slot, length):
            pass

        def close(self, slot):
            del self.held[slot]

        def flush(self):
            pass

        def tokens_held(self):
            return sum(self.held.values())

        def layer(self, index):
            return LatentLayerView(self.data[index])

        def check(self):
            assert all(0 <= n <= self.sizes.max_seq_len for n in self.held.values())

    @dataclass(frozen=True)
    class LatentSpec:
        rank: int

        def make_store(self, n_layers, sizes, dtype, device, allocate=True):
            return LatentStore(self, n_layers, sizes, device, allocate)

    # ---- the parts ------------------------------------------------------------
    @register_part("mixer", "toy_prefix_mean")
    class PrefixMean(Mixer):
        """c_t = x_t A^T (``rank`` numbers per token, kept); y_t = mean(c_0..c_t) B^T."""

        def __init__(self, ctx, width, rank):
            super().__init__(ctx)
            self.width, self.rank = width, rank

        def param_specs(self):
            return {"down.weight": ParamSpec((self.rank, self.width)),
                    "up.weight": ParamSpec((self.width, self.rank))}

        def load(self, params):
            self.down_w, self.up_w = params["down.weight"], params["up.weight"]

        def cache_spec(self):
            return LatentSpec(self.rank)

        def captures_prompts(self):
            return True                  # device arrays only, below

        def forward(self, x, step, cache):
            store = cache.latent                                    # [slots + 1, L, rank]
            spare, L = store.shape[0] - 1, store.shape[1]
            slot = step.slots.long()[step.token_seq.long()]
            slot = torch.where(slot < 0, torch.full_like(slot, spare), slot)
            pos = step.token_pos.long()
            c = x.float() @ self.down_w.float().T
            store[slot, pos] = c                                    # first every row of the step ...
            seen = store[slot]                                      # ... then each row reads its prefix
            mask = (torch.arange(L, device=x.device)[None, :] <= pos[:, None]).unsqueeze(-1)
            mean = (seen * mask).sum(1) / (pos[:, None] + 1).float()
            return (mean @ self.up_w.float().T).to(x.dtype)

    @register_part("embedding", "toy_token_plus_position")
    class TokenPlusPosition(Embedding):
        """x_t = E[token_t] + P[position_t]: an encoding added to the embeddings is
        an embedding part; the step says where every row stands."""

        def __init__(self, ctx, vocab, hidden, max_positions):
            super().__init__(ctx)
            self.vocab, self.hidden, self.max_positions = vocab, hidden, max_positions

        def param_specs(self):
            return {"weight": ParamSpec((self.vocab, self.hidden)),
                    "positions.weight": ParamSpec((self.max_positions, self.hidden))}

        def load(self, params):
            self.weight, self.positions = params["weight"], params["positions.weight"]

        def captures_prompts(self):
            return True

        def forward(self, tokens, step):
            x = self.weight[tokens.long()].float() + self.positions[step.token_pos.long()].float()
            return x.to(self.ctx.dtype)

    def plan(cfg):
        norm = PartSpec("rmsnorm", dict(dim=cfg.width, eps=cfg.eps))
        ffn = PartSpec("swiglu", dict(hidden=cfg.width, intermediate=cfg.inner))
        attn = PartSpec("gqa_attention", dict(
            hidden=cfg.width, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
            position=PartSpec("rotary_half_split", dict(head_dim=cfg.head_dim, theta=cfg.theta)),
            qk_norm_eps=cfg.eps))
        mixers = [PartSpec("toy_prefix_mean", dict(width=cfg.width, rank=cfg.rank)), attn,
                  PartSpec("toy_prefix_mean", dict(width=cfg.width, rank=cfg.rank))]
        roles = {"norm1": "n1.", "mixer": "mixer.", "norm2": "n2.", "feedforward": "ffn."}
        layers = tuple(LayerPlan(PartSpec("prenorm", dict(norm1=norm, mixer=m, norm2=norm,
                                                          feedforward=ffn)), f"blocks.{i}.", roles)
                       for i, m in enumerate(mixers))
        return ModelPlan(
            embedding=PartSpec("toy_token_plus_position",
                               dict(vocab=cfg.vocab, hidden=cfg.width, max_positions=cfg.max_positions)),
            embedding_prefix="embed.", layers=layers,
            schedule=tuple(ScheduleEntry(i) for i in range(3)), final_norm=norm,
            final_norm_prefix="final.",
            head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=cfg.width, tied=False)),
            head_prefix="head.", vocab_size=cfg.vocab, max_position=cfg.max_positions)

    register_architecture("ToyLatentForCausalLM", ToyConfig, plan, model_types=("toy_latent",))


def _oracle(w, cfg, tokens):
    """The toy model, whole sequence, 64-bit."""
    T = len(tokens)
    x = plain.embed(w["embed.weight"], tokens) + w["embed.positions.weight"].double()[:T]
    pos = list(range(T))
    D, nq, nkv = cfg["head_dim"], cfg["heads"], cfg["kv_heads"]
    for layer in range(3):
        p = f"blocks.{layer}."
        n = plain.rms_norm(x, w[p + "n1.weight"], cfg["eps"])
        if layer == 1:
            q = (n @ w[p + "mixer.q_proj.weight"].double().T).reshape(T, nq, D)
            k = (n @ w[p + "mixer.k_proj.weight"].double().T).reshape(T, nkv, D)
            v = (n @ w[p + "mixer.v_proj.weight"].double().T).reshape(T, nkv, D)
            q = plain.rms_norm(q, w[p + "mixer.q_norm.weight"], cfg["eps"])
            k = plain.rms_norm(k, w[p + "mixer.k_norm.weight"], cfg["eps"])
            cos, sin = plain.rope_cos_sin(pos, D, cfg["theta"])
            o = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v)
            a = o.reshape(T, nq * D) @ w[p + "mixer.o_proj.weight"].double().T
        else:
            c = n @ w[p + "mixer.down.weight"].double().T
            mean = torch.cumsum(c, 0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
            a = mean @ w[p + "mixer.up.weight"].double().T
        x = x + a
        m = plain.rms_norm(x, w[p + "n2.weight"], cfg["eps"])
        x = x + plain.swiglu(m, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"],
                             w[p + "ffn.down_proj.weight"])
    return plain.rms_norm(x, w["final.weight"], cfg["eps"]) @ w["head.weight"].double().T


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from safetensors import safe_open
    from grout_b200.config import unregister_architecture
    from grout_b200.parts import unregister_part
    from grout_b200.weights import write_random_model
    _register()
    d = str(tmp_path_factory.mktemp("toy_latent"))
    write_random_model(TOY, 8, d)
    with safe_open(os.path.join(d, "model.safetensors"), "pt") as f:
        w = {k: f.get_tensor(k) for k in f.keys()}
    yield d, w
    unregister_architecture("ToyLatentForCausalLM")
    unregister_part("mixer", "toy_prefix_mean")
    unregister_part("embedding", "toy_token_plus_position")


def test_the_cache_holds_a_store_it_has_never_heard_of(toy):
    from grout_b200.cache import SequenceCache
    from grout_b200.config import load_config
    from grout_b200.engine.model import Model
    from grout_b200.parts import BuildContext
    d, w = toy
    arch, cfg = load_config(d)
    m = Model(arch.plan(cfg), BuildContext(torch.bfloat16, torch.device("cpu")))
    assert set(m.expected()) == set(w)
    lay = m.cache_layout()
    assert [type(s).__name__ for s, _ in lay.groups] == ["LatentSpec", "KVSpec"]
    assert lay.groups[0][1] == [0, 2] and lay.groups[1][1] == [1]
    assert m.captures_prompts()
    cache = SequenceCache(lay, max_tokens=256, max_slots=3, max_seq_len=128, dtype=torch.bfloat16,
                          device="cpu", allocate=False)
    a, b = cache.open(), cache.open()
    cache.reserve(a, 70), cache.advance(a, 70), cache.reserve(b, 5), cache.advance(b, 5)
    assert type(cache.stores[0]).__name__ == "LatentStore" and cache.stores[0].tokens_held() == 75
    cache.check()
    cache.close(a), cache.close(b)
    cache.check()
    assert cache.stores[0].tokens_held() == 0 and cache.tokens_held() == 0

    class NoStore:
        pass
    with pytest.raises(TypeError, match="make_store"):
        SequenceCache(type(lay)([(NoStore(), [0])], {0: (0, 0)}), max_tokens=64, max_slots=1,
                      max_seq_len=64, dtype=torch.bfloat16, device="cpu", allocate=False)


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_toy_model_steps_in_every_cut(toy, dtype, graphs):
    from grout_b200.engine import Engine
    d, w = toy
    eng = Engine.load(d, dtype=dtype, max_tokens=2048, max_batch=4, use_graphs=graphs)
    reqs = [random_tokens(n, TOY["vocab"], 950 + n) for n in (75, 9, 40)]
    want = [_oracle(w, TOY, r) for r in reqs]
    assert_close(run_whole(eng, reqs[0]), want[0], dtype, "latent toy whole")
    assert_close(run_tail_decoded(eng, reqs[0], tail=20), want[0], dtype, "latent toy tail decoded")
    assert_close(run_chunks(eng, reqs[0], [10, 1, 60, 4]), want[0], dtype, "latent toy in chunks")
    for _ in range(2):                                   # twice: a reused slot's old latents are not read
        got = run_batch(eng, reqs, [60, 2, 33])
        for g, x in zip(got, want):
            assert_close(g, x, dtype, "latent toy batch")
    eng.cache.check()
    # the toy parts allow capture, so prompt steps ran as graphs when graphs are on
    assert bool(eng.graphs.prompt_graphs) == graphs and bool(eng.graphs.decode_graphs) == graphs
