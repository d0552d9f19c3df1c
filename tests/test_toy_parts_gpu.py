"""Parts and an architecture defined here, in the test, and run by the library
without a change to its files: a mixer with fixed-size state of its own, a layer
that runs twice, and an attention layer that reads another layer's cache.
The toy model is nobody's architecture; it only shows the interfaces."""
import os
from dataclasses import dataclass

import pytest
import torch

from conftest import random_tokens
from helpers import assert_close, run_batch, run_tail_decoded, run_whole
from plain import qwen3 as plain

pytestmark = pytest.mark.gpu

TOY = dict(architectures=["ToyStateForCausalLM"], model_type="toy_state", vocab=97, width=48,
           inner=80, heads=4, kv_heads=2, head_dim=16, decay=0.75, eps=1e-5, theta=300.0,
           max_positions=200)


def _register():
    from grout_b200.cache import StateSpec
    from grout_b200.config import register_architecture
    from grout_b200.config.base import ModelConfig
    from grout_b200.parts import (LayerPlan, Linear, Mixer, ModelPlan, ParamSpec, PartSpec,
                                  ScheduleEntry, register_part)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab: int
        width: int
        inner: int
        heads: int
        kv_heads: int
        head_dim: int
        decay: float
        eps: float
        theta: float
        max_positions: int
        model_type: str = "toy_state"
        architectures: tuple = ("ToyStateForCausalLM",)

    @register_part("mixer", "toy_decay_state")
    class DecayState(Mixer):
        """s_t = decay * s_{t-1} + x_t per sequence, y_t = s_t W^T.  The state is
        one vector per sequence; it is written with library tensor operations,
        which a test may use."""

        def __init__(self, ctx, width, decay):
            super().__init__(ctx)
            self.width, self.decay = width, decay

        def param_specs(self):
            return {"mix.weight": ParamSpec((self.width, self.width))}

        def load(self, params):
            self.mix = Linear(params["mix.weight"])

        def kernel_modules(self):
            return self.mix.kernel_modules()

        def cache_spec(self):
            return StateSpec((self.width,), torch.float32)

        def forward(self, x, step, cache):
            state = cache.state                                  # [slots + 1, width]
            scratch = state.shape[0] - 1
            slot = torch.where(step.slots < 0, torch.full_like(step.slots, scratch), step.slots).long()
            xf = x.float()
            if step.decode:                                      # one row per sequence
                s = self.decay * state[slot] + xf
                state[slot] = s
                out = s
            else:                                                # rows of a sequence in order
                out = torch.empty_like(xf)
                o = 0
                for i, n in enumerate(step.q_lens):
                    s = state[slot[i]].clone()
                    for t in range(n):
                        s = self.decay * s + xf[o + t]
                        out[o + t] = s
                    state[slot[i]] = s
                    o += n
            return self.mix(out.to(x.dtype))

    def plan(cfg):
        norm = PartSpec("rmsnorm", dict(dim=cfg.width, eps=cfg.eps))
        ffn = PartSpec("swiglu", dict(hidden=cfg.width, intermediate=cfg.inner))
        pos = PartSpec("rotary_half_split", dict(head_dim=cfg.head_dim, theta=cfg.theta))
        attn = dict(hidden=cfg.width, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads,
                    head_dim=cfg.head_dim, position=pos, qk_norm_eps=cfg.eps)
        mixers = [PartSpec("gqa_attention", attn),
                  PartSpec("toy_decay_state", dict(width=cfg.width, decay=cfg.decay)),
                  PartSpec("gqa_attention", dict(attn, shares_kv=True))]
        roles = {"norm1": "n1.", "mixer": "mixer.", "norm2": "n2.", "feedforward": "ffn."}
        layers = tuple(LayerPlan(PartSpec("prenorm", dict(norm1=norm, mixer=m, norm2=norm,
                                                          feedforward=ffn)), f"blocks.{i}.", roles)
                       for i, m in enumerate(mixers))
        # layer 0 attends and stores; layer 1 carries state; layer 2 reads layer 0's keys
        # and values; then layers 1 and 0 run once more, each with a cache of its own
        schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, cache_of=0),
                    ScheduleEntry(1), ScheduleEntry(0))
        return ModelPlan(embedding=PartSpec("token", dict(vocab=cfg.vocab, hidden=cfg.width)),
                         embedding_prefix="embed.", layers=layers, schedule=schedule,
                         final_norm=norm, final_norm_prefix="final.",
                         head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=cfg.width, tied=True)),
                         head_prefix="head.", vocab_size=cfg.vocab, max_position=cfg.max_positions)

    register_architecture("ToyStateForCausalLM", ToyConfig, plan, model_types=("toy_state",))


def _toy_oracle(w, cfg, tokens):
    """The toy model, whole sequence, 64-bit, from the plain parts."""
    T = len(tokens)
    x = plain.embed(w["embed.weight"], tokens)
    pos = list(range(T))
    D, nq, nkv = cfg["head_dim"], cfg["heads"], cfg["kv_heads"]

    def project_kv(n, p):
        k = (n @ w[p + "mixer.k_proj.weight"].double().T).reshape(T, nkv, D)
        v = (n @ w[p + "mixer.v_proj.weight"].double().T).reshape(T, nkv, D)
        k = plain.rms_norm(k, w[p + "mixer.k_norm.weight"], cfg["eps"])
        cos, sin = plain.rope_cos_sin(pos, D, cfg["theta"])
        return plain.apply_rope(k, cos, sin), v

    def attend(n, p, kv):
        q = (n @ w[p + "mixer.q_proj.weight"].double().T).reshape(T, nq, D)
        q = plain.rms_norm(q, w[p + "mixer.q_norm.weight"], cfg["eps"])
        cos, sin = plain.rope_cos_sin(pos, D, cfg["theta"])
        o = plain.causal_attention(plain.apply_rope(q, cos, sin), kv[0], kv[1])
        return o.reshape(T, nq * D) @ w[p + "mixer.o_proj.weight"].double().T

    def state_mixer(n, p):
        s = torch.zeros(n.shape[1], dtype=torch.float64)
        out = torch.empty_like(n)
        for t in range(T):
            s = cfg["decay"] * s + n[t]
            out[t] = s
        return out @ w[p + "mixer.mix.weight"].double().T

    kv0 = None
    for layer, shared in [(0, False), (1, False), (2, True), (1, False), (0, False)]:
        p = f"blocks.{layer}."
        n = plain.rms_norm(x, w[p + "n1.weight"], cfg["eps"])
        if layer == 1:
            a = state_mixer(n, p)
        elif shared:
            a = attend(n, p, kv0)
        else:
            kv = project_kv(n, p)
            if kv0 is None:
                kv0 = kv
            a = attend(n, p, kv)
        x = x + a
        m = plain.rms_norm(x, w[p + "n2.weight"], cfg["eps"])
        x = x + plain.swiglu(m, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"],
                             w[p + "ffn.down_proj.weight"])
    return plain.rms_norm(x, w["final.weight"], cfg["eps"]) @ w["embed.weight"].double().T


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from safetensors import safe_open
    from grout_b200.config import unregister_architecture
    from grout_b200.parts import unregister_part
    from grout_b200.weights import write_random_model
    _register()
    d = str(tmp_path_factory.mktemp("toy"))
    write_random_model(TOY, 6, d)
    with safe_open(os.path.join(d, "model.safetensors"), "pt") as f:
        w = {k: f.get_tensor(k) for k in f.keys()}
    yield d, w
    unregister_architecture("ToyStateForCausalLM")
    unregister_part("mixer", "toy_decay_state")


def test_toy_layout(toy):
    from grout_b200.config import load_config
    from grout_b200.engine.model import Model
    from grout_b200.parts import BuildContext
    d, w = toy
    arch, cfg = load_config(d)
    assert arch.name == "ToyStateForCausalLM"
    m = Model(arch.plan(cfg), BuildContext(torch.bfloat16, torch.device("cpu")))
    assert set(m.expected()) == set(w)
    assert "blocks.2.mixer.k_proj.weight" not in w        # the reading layer projects no keys
    lay = m.cache_layout()
    # entries 0 and 4 own keys and values (one store, two layers), 1 and 3 own state, 2 owns nothing
    assert [type(s).__name__ for s, _ in lay.groups] == ["KVSpec", "StateSpec"]
    assert lay.groups[0][1] == [0, 4] and lay.groups[1][1] == [1, 3] and 2 not in lay.where


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_steps_in_every_cut(toy, dtype, graphs):
    from grout_b200.engine import Engine
    d, w = toy
    eng = Engine.load(d, dtype=dtype, max_tokens=2048, max_batch=4, use_graphs=graphs)
    reqs = [random_tokens(n, TOY["vocab"], 900 + n) for n in (70, 9, 33)]
    want = [_toy_oracle(w, TOY, r) for r in reqs]
    assert_close(run_whole(eng, reqs[0]), want[0], dtype, "toy whole")
    assert_close(run_tail_decoded(eng, reqs[0], tail=20), want[0], dtype, "toy tail decoded")
    for _ in range(2):                                   # twice: state of a reused slot starts at zero
        got = run_batch(eng, reqs, [50, 2, 33 - 8])
        for g, x in zip(got, want):
            assert_close(g, x, dtype, "toy batch")
    eng.cache.check()
