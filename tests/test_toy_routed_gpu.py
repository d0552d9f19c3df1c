"""More toy parts defined here, in the test, and run by the library without a
change to its files: a feed-forward that routes every token to two of four
small experts, a position encoding with arithmetic of its own (a rotation of
adjacent pairs, applied outside the fused kernel), a norm without a fused kernel
(mean-centred, with a bias), and a layer whose attention sees a window.
The toy model is nobody's architecture; it only shows the interfaces."""
import math
import os
from dataclasses import dataclass

import pytest
import torch

from conftest import random_tokens
from helpers import assert_close, run_batch, run_tail_decoded, run_whole
from plain import qwen3 as plain

pytestmark = pytest.mark.gpu

TOY = dict(architectures=["ToyRoutedForCausalLM"], model_type="toy_routed", vocab=131, width=40,
           inner=24, experts=4, picked=2, heads=5, kv_heads=1, head_dim=16, eps=1e-4, theta=50.0,
           window=24, max_positions=160)


def _register():
    from grout_b200.config import register_architecture
    from grout_b200.config.base import ModelConfig
    from grout_b200.parts import (LayerPlan, Linear, ModelPlan, ParamSpec, PartSpec, ScheduleEntry,
                                  register_part)
    from grout_b200.parts.feedforward import FeedForward
    from grout_b200.parts.norm import Norm
    from grout_b200.parts.position import PositionEncoding

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab: int
        width: int
        inner: int
        experts: int
        picked: int
        heads: int
        kv_heads: int
        head_dim: int
        eps: float
        theta: float
        window: int
        max_positions: int
        model_type: str = "toy_routed"
        architectures: tuple = ("ToyRoutedForCausalLM",)

    @register_part("feedforward", "toy_routed")
    class Routed(FeedForward):
        """Router logits and their softmax in 32-bit, the best ``picked`` experts
        of a token (the first of equals), their weights renormalised to sum 1;
        expert e is relu(x U_e^T) D_e^T.  Routing uses library tensor operations,
        which a test may; the experts' products are the library's ``Linear``."""

        def __init__(self, ctx, width, inner, experts, picked):
            super().__init__(ctx)
            self.width, self.inner, self.n, self.k = width, inner, experts, picked

        def param_specs(self):
            specs = {"router.weight": ParamSpec((self.n, self.width))}
            for e in range(self.n):
                specs[f"experts.{e}.up.weight"] = ParamSpec((self.inner, self.width))
                specs[f"experts.{e}.down.weight"] = ParamSpec((self.width, self.inner))
            return specs

        def load(self, params):
            self.router = params["router.weight"].float()
            self.up = [Linear(params[f"experts.{e}.up.weight"]) for e in range(self.n)]
            self.down = [Linear(params[f"experts.{e}.down.weight"]) for e in range(self.n)]

        def kernel_modules(self):
            return self.up[0].kernel_modules()

        def forward(self, x, step):
            probs = torch.softmax(x.float() @ self.router.T, dim=-1)
            top, idx = torch.topk(probs, self.k, dim=-1)         # ties: the lower index first
            top = top / top.sum(dim=-1, keepdim=True)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.n):
                gate = (top * (idx == e)).sum(dim=-1, keepdim=True)   # 0 where e was not picked
                # every expert sees every row (the rows' packing is the step's); rows that
                # did not pick it are multiplied by 0
                h = torch.relu(self.up[e](x).float()).to(x.dtype)
                out += gate * self.down[e](h).float()
            return out.to(x.dtype)

    @register_part("position", "toy_pair_rotation")
    class PairRotation(PositionEncoding):
        """Rotates the adjacent pairs (2j, 2j+1) of every query and key head by
        pos * theta^(-j / (D/2)); arithmetic of its own, so attention applies it
        between its projection and the cache write."""

        def __init__(self, ctx, head_dim, theta):
            super().__init__(ctx)
            j = torch.arange(head_dim // 2, dtype=torch.float32)
            self.inv = (theta ** (-j / (head_dim // 2))).to(ctx.device)

        def apply_qk(self, q, k, token_pos):
            ang = token_pos.float()[:, None] * self.inv[None, :]          # [T, D/2]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

            def rot(x):
                if x.shape[1] == 0:
                    return x
                xf = x.float()
                a, b = xf[..., 0::2], xf[..., 1::2]
                y = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1)
                return y.reshape(x.shape).to(x.dtype)
            return rot(q), rot(k)

    @register_part("norm", "toy_centred")
    class Centred(Norm):
        """(x - mean) / sqrt(var + eps) * w + b in 32-bit; it has no fused kernel, so
        the family's default adds the residual first and then calls ``forward``."""

        def __init__(self, ctx, dim, eps):
            super().__init__(ctx)
            self.dim, self.eps = dim, eps

        def param_specs(self):
            return {"weight": ParamSpec((self.dim,), "vector"), "bias": ParamSpec((self.dim,), "vector")}

        def load(self, params):
            self.w, self.b = params["weight"].float(), params["bias"].float()

        def kernel_modules(self):
            return ("elementwise",)

        def forward(self, x):
            xf = x.float()
            xc = xf - xf.mean(dim=-1, keepdim=True)
            y = xc / torch.sqrt((xc * xc).mean(dim=-1, keepdim=True) + self.eps) * self.w + self.b
            return y.to(self.ctx.dtype)

    def plan(cfg):
        rms = PartSpec("rmsnorm", dict(dim=cfg.width, eps=cfg.eps))
        centred = PartSpec("toy_centred", dict(dim=cfg.width, eps=cfg.eps))
        routed = PartSpec("toy_routed", dict(width=cfg.width, inner=cfg.inner, experts=cfg.experts,
                                             picked=cfg.picked))
        dense = PartSpec("swiglu", dict(hidden=cfg.width, intermediate=cfg.inner))
        attn = dict(hidden=cfg.width, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads, head_dim=cfg.head_dim)
        pair = PartSpec("toy_pair_rotation", dict(head_dim=cfg.head_dim, theta=cfg.theta))
        half = PartSpec("rotary_half_split", dict(head_dim=cfg.head_dim, theta=cfg.theta, rot_dim=8))
        blocks = [
            # all keys, pair rotation, no q/k norm, centred norms, routed feed-forward
            dict(norm1=centred, mixer=PartSpec("gqa_attention", dict(attn, position=pair)),
                 norm2=centred, feedforward=routed),
            # a window of keys, half-split rotation of the first 8 elements, q/k norm, dense
            dict(norm1=rms, mixer=PartSpec("gqa_attention", dict(attn, position=half, qk_norm_eps=cfg.eps,
                                                                 window=cfg.window)),
                 norm2=rms, feedforward=dense),
            # no position encoding at all, routed again
            dict(norm1=rms, mixer=PartSpec("gqa_attention", dict(attn, position=PartSpec("none", {}),
                                                                 scale=0.2)),
                 norm2=centred, feedforward=routed),
        ]
        roles = {"norm1": "n1.", "mixer": "mixer.", "norm2": "n2.", "feedforward": "ffn."}
        layers = tuple(LayerPlan(PartSpec("prenorm", b), f"blocks.{i}.", roles) for i, b in enumerate(blocks))
        return ModelPlan(embedding=PartSpec("token", dict(vocab=cfg.vocab, hidden=cfg.width)),
                         embedding_prefix="embed.", layers=layers,
                         schedule=tuple(ScheduleEntry(i) for i in range(3)),
                         final_norm=centred, final_norm_prefix="final.",
                         head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=cfg.width, tied=False)),
                         head_prefix="head.", vocab_size=cfg.vocab, max_position=cfg.max_positions)

    register_architecture("ToyRoutedForCausalLM", ToyConfig, plan, model_types=("toy_routed",))


def _oracle(w, cfg, tokens):
    """The toy model, whole sequence, 64-bit.  Returns the logits and, per token,
    the smallest gap between the last expert picked and the first one left out."""
    T = len(tokens)
    D, nq, nkv = cfg["head_dim"], cfg["heads"], cfg["kv_heads"]
    pos = torch.arange(T, dtype=torch.float64)

    def centred(x, p):
        xc = x - x.mean(dim=-1, keepdim=True)
        return xc / torch.sqrt((xc * xc).mean(dim=-1, keepdim=True) + cfg["eps"]) * w[p + "weight"].double() \
            + w[p + "bias"].double()

    def rms(x, p):
        return plain.rms_norm(x, w[p + "weight"], cfg["eps"])

    def pair_rotation(x):
        j = torch.arange(D // 2, dtype=torch.float32)
        inv = (cfg["theta"] ** (-j / (D // 2))).double()       # the part computes it in 32-bit
        ang = (pos.float()[:, None] * inv.float()[None, :]).double()
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b = x[..., 0::2], x[..., 1::2]
        return torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).reshape(x.shape)

    def attention(n, p, kind):
        q = (n @ w[p + "q_proj.weight"].double().T).reshape(T, nq, D)
        k = (n @ w[p + "k_proj.weight"].double().T).reshape(T, nkv, D)
        v = (n @ w[p + "v_proj.weight"].double().T).reshape(T, nkv, D)
        window = None
        if kind == 0:
            q, k = pair_rotation(q), pair_rotation(k)
        elif kind == 1:
            q = plain.rms_norm(q, w[p + "q_norm.weight"], cfg["eps"])
            k = plain.rms_norm(k, w[p + "k_norm.weight"], cfg["eps"])
            cos, sin = plain.rope_cos_sin(list(range(T)), 8, cfg["theta"])
            q = torch.cat([plain.apply_rope(q[..., :8], cos, sin), q[..., 8:]], dim=-1)
            k = torch.cat([plain.apply_rope(k[..., :8], cos, sin), k[..., 8:]], dim=-1)
            window = cfg["window"]
        else:
            q = q * (0.2 * math.sqrt(D))          # scores q.k * 0.2 instead of q.k / sqrt(D)
        o = plain.causal_attention(q, k, v, window=window)
        return o.reshape(T, nq * D) @ w[p + "o_proj.weight"].double().T

    margins = torch.full((T,), 1.0, dtype=torch.float64)

    def routed(m, p):
        probs = torch.softmax(m @ w[p + "router.weight"].double().T, dim=-1)
        ranked = probs.sort(dim=-1, descending=True).values
        margins.copy_(torch.minimum(margins, ranked[:, cfg["picked"] - 1] - ranked[:, cfg["picked"]]))
        top, idx = torch.topk(probs, cfg["picked"], dim=-1)
        top = top / top.sum(dim=-1, keepdim=True)
        out = torch.zeros_like(m)
        for t in range(T):
            for g, e in zip(top[t], idx[t]):
                e = int(e)
                h = torch.relu(m[t] @ w[p + f"experts.{e}.up.weight"].double().T)
                out[t] += g * (h @ w[p + f"experts.{e}.down.weight"].double().T)
        return out

    x = plain.embed(w["embed.weight"], tokens)
    for i in range(3):
        p = f"blocks.{i}."
        n = centred(x, p + "n1.") if i == 0 else rms(x, p + "n1.")
        x = x + attention(n, p + "mixer.", i)
        m = rms(x, p + "n2.") if i == 1 else centred(x, p + "n2.")
        if i == 1:
            x = x + plain.swiglu(m, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"],
                                 w[p + "ffn.down_proj.weight"])
        else:
            x = x + routed(m, p + "ffn.")
    return centred(x, "final.") @ w["head.weight"].double().T, margins


def _assert_close_where_routing_is_clear(got, want, margins, dtype, what):
    """In bf16 a token whose experts are nearly tied may pick the other one; that
    is rounding of the router's input, not a fault of a cache or a batch, and such
    rows (few) are left out.  In 32-bit every row is compared."""
    if dtype == "bfloat16":
        clear = margins > 3e-4          # some ten times what bf16 rounding moves a probability here
        assert int(clear.sum()) >= 0.9 * len(margins), "the test's weights make routing a coin toss"
        got, want = got[clear], want[clear]
    assert_close(got, want, dtype, what)


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from safetensors import safe_open
    from grout_b200.config import unregister_architecture
    from grout_b200.parts import unregister_part
    from grout_b200.weights import write_random_model
    _register()
    d = str(tmp_path_factory.mktemp("toy_routed"))
    write_random_model(TOY, 8, d)
    with safe_open(os.path.join(d, "model.safetensors"), "pt") as f:
        w = {k: f.get_tensor(k) for k in f.keys()}
    yield d, w
    unregister_architecture("ToyRoutedForCausalLM")
    unregister_part("feedforward", "toy_routed")
    unregister_part("position", "toy_pair_rotation")
    unregister_part("norm", "toy_centred")


def test_layout_has_a_store_for_all_keys_and_one_for_the_window(toy):
    from grout_b200.config import load_config
    from grout_b200.engine.model import Model
    from grout_b200.parts import BuildContext
    d, w = toy
    arch, cfg = load_config(d)
    m = Model(arch.plan(cfg), BuildContext(torch.bfloat16, torch.device("cpu")))
    assert set(m.expected()) == set(w)
    assert "blocks.0.ffn.experts.3.down.weight" in w and "blocks.0.mixer.q_norm.weight" not in w
    lay = m.cache_layout()
    assert [(s.window, layers) for s, layers in lay.groups] == [(None, [0, 2]), (TOY["window"], [1])]


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_toy_model_steps_in_every_cut(toy, dtype, graphs):
    from grout_b200.engine import Engine
    d, w = toy
    eng = Engine.load(d, dtype=dtype, max_tokens=2048, max_batch=4, use_graphs=graphs)
    reqs = [random_tokens(n, TOY["vocab"], 950 + n) for n in (90, 7, 41)]
    want = [_oracle(w, TOY, r) for r in reqs]
    check = _assert_close_where_routing_is_clear
    check(run_whole(eng, reqs[0]), *want[0], dtype, "routed toy whole")
    check(run_tail_decoded(eng, reqs[0], tail=30), *want[0], dtype, "routed toy tail decoded")
    for _ in range(2):
        got = run_batch(eng, reqs, [60, 3, 41 - 9])
        for g, (x, margins) in zip(got, want):
            check(g, x, margins, dtype, "routed toy batch")
    eng.cache.check()
    outs = eng.generate([reqs[1], reqs[2]], 6, ignore_eos=True)
    assert all(len(o.token_ids) == 6 for o in outs) and eng.cache.slots.n_held == 0
