"""Parts and an architecture defined HERE, in the test, registered and run without a change
to the library: a mixer with fixed-size state of its own (no keys, no values), a run order
that names a layer twice and lets an entry read another entry's cache, a plain pre-norm
arrangement.  Stepping token by token must give what whole prompts give, and both must give
what a few lines of PyTorch on whole sequences give."""
import math
import random
from dataclasses import dataclass

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _register():
    from hos_b200 import ops
    from hos_b200.config.base import LayerCall, LayerSpec, ModelConfig, ModelPlan, PartSpec
    from hos_b200.parts import linear
    from hos_b200.parts.base import Mixer, StateNeed, WeightSpec
    from hos_b200.registry import register_architecture, register_part

    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + h_t (per sequence, state [width] float32); y_t = W s_t."""

        def __init__(self, spec, rt):
            super().__init__(spec, rt)
            self.width, self.decay = int(spec.params["width"]), float(spec.params["decay"])

        def weight_specs(self):
            return [WeightSpec(self.spec.weights["w"], (self.width, self.width), "matrix", 0.05)]

        def bind(self, tensors):
            self.w = self._matrix(tensors[self.spec.weights["w"]])

        def state_needs(self):
            return [StateNeed("s", (self.width,), torch.float32)]

        def forward(self, h, step, store):
            state = store.state["s"]
            out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
            for i, slot in enumerate(step.slots_host):
                lo, hi = step.cu_host[i], step.cu_host[i + 1]
                s = state[slot]
                for r in range(lo, hi):
                    s = self.decay * s + h[r].float()
                    out[r] = s
                state[slot] = s
            return linear.matmul(out.to(h.dtype), self.w)

    register_part("mixer", "toy_decay", DecayMixer)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        width: int
        vocab: int
        inner: int
        decay: float
        architecture = "ToyForTests"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["width"], raw["vocab"], raw["inner"], raw["decay"])

        def to_dict(self):
            return dict(architectures=["ToyForTests"], width=self.width, vocab=self.vocab, inner=self.inner,
                        decay=self.decay, vocab_size=self.vocab)

    def plan(cfg):
        D = cfg.width
        def norm(n):
            return PartSpec("rmsnorm", {"width": D, "eps": 1e-5, "add_one": False}, {"weight": n})
        def ffn(p):
            return PartSpec("gated_mlp", {"width": D, "inner": cfg.inner, "activation": "silu"},
                            {"gate": p + "g", "up": p + "u", "down": p + "d"})
        attn = PartSpec("softmax_attention",
                        {"width": D, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16, "scale": 0.25, "softcap": 0.0,
                         "window": None,
                         "position": PartSpec("rotary", {"theta": 100.0, "rotary_dim": 8, "style": "interleaved"})},
                        {"q": "l0.q", "k": "l0.k", "v": "l0.v", "o": "l0.o"})
        decay = PartSpec("toy_decay", {"width": D, "decay": cfg.decay}, {"w": "l1.w"})
        layers = [LayerSpec("prenorm", attn, ffn("l0."), {"pre_mixer": norm("l0.n1"), "pre_ffn": norm("l0.n2")}),
                  LayerSpec("prenorm", decay, ffn("l1."), {"pre_mixer": norm("l1.n1"), "pre_ffn": norm("l1.n2")})]
        # attention layer, decay layer, the attention layer AGAIN reading the first call's cache,
        # and the decay layer again (shared weights, state of its own)
        schedule = [LayerCall(0), LayerCall(1), LayerCall(0, cache_from=0), LayerCall(1)]
        return ModelPlan(D, cfg.vocab, 512, PartSpec("scaled_embedding", {"vocab": cfg.vocab, "width": D, "scale": 1.0},
                                                     {"table": "emb"}),
                         layers, schedule, norm("final"),
                         PartSpec("linear_head", {"vocab": cfg.vocab, "width": D, "softcap": 0.0},
                                  {"table": "head", "tied_to": "emb"}))

    register_architecture("ToyForTests", ToyConfig, plan)
    return ToyConfig


def _plain_toy(w, cfg, tokens):
    """The toy model on one whole sequence, in float32 PyTorch."""
    D, T = cfg.width, len(tokens)
    def norm(x, n):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w[n]
    def ffn(h, p):
        g = h @ w[p + "g"].T
        return ((g / (1 + torch.exp(-g))) * (h @ w[p + "u"].T)) @ w[p + "d"].T
    def rope(v):
        i = torch.arange(4, dtype=torch.float32)
        ang = torch.arange(T, dtype=torch.float32)[:, None] * (1.0 / torch.pow(torch.tensor(100.0), 2 * i / 8))[None]
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        out = v.clone()
        a, b = v[..., 0:8:2], v[..., 1:8:2]
        out[..., 0:8:2], out[..., 1:8:2] = a * c - b * s, a * s + b * c
        return out
    def attention(h, kv=None):
        q = rope((h @ w["l0.q"].T).view(T, 2, 16))
        if kv is None:
            kv = (rope((h @ w["l0.k"].T).view(T, 1, 16)), (h @ w["l0.v"].T).view(T, 1, 16))
        k, v = kv
        mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
        out = torch.empty(T, 2, 16)
        for hh in range(2):
            s = (q[:, hh] @ k[:, 0].T) * 0.25
            out[:, hh] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, 0]
        return out.reshape(T, 32) @ w["l0.o"].T, kv
    def decay(h):
        s, rows = torch.zeros(D), []
        for t in range(T):
            s = cfg.decay * s + h[t]
            rows.append(s)
        return torch.stack(rows) @ w["l1.w"].T
    x = w["emb"][torch.tensor(tokens)]
    a, kv = attention(norm(x, "l0.n1"))
    x = x + a
    x = x + ffn(norm(x, "l0.n2"), "l0.")
    x = x + decay(norm(x, "l1.n1"))
    x = x + ffn(norm(x, "l1.n2"), "l1.")
    a, _ = attention(norm(x, "l0.n1"), kv)            # same weights, the FIRST call's keys and values
    x = x + a
    x = x + ffn(norm(x, "l0.n2"), "l0.")
    x = x + decay(norm(x, "l1.n1"))                   # same weights, a state of its own
    x = x + ffn(norm(x, "l1.n2"), "l1.")
    return norm(x, "final") @ w["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_stateful_mixer_steps_like_whole_prompts(dtype):
    from hos_b200.engine import Runner
    from hos_b200.model import weight_specs_for
    from hos_b200.weights import RandomSource
    ToyConfig = _register()
    cfg = ToyConfig(width=48, vocab=101, inner=80, decay=0.8)
    specs = weight_specs_for(cfg)
    src = RandomSource(specs, 5)
    r = Runner(cfg, src, dtype=dtype, max_tokens=2048)
    assert len(r.cache.groups) == 1 and r.cache.groups[0].n_entries == 1      # one cache, read twice
    assert set(r.cache.stores[1].state) == {"s"} and set(r.cache.stores[3].state) == {"s"}
    assert r.cache.stores[1].state["s"].data_ptr() != r.cache.stores[3].state["s"].data_ptr()
    w = {n: src.read(n).float() for n in src.names()}
    rng = random.Random(0)
    seqs = [[rng.randrange(101) for _ in range(n)] for n in (30, 7, 75)]
    want = [_plain_toy(w, cfg, s) for s in seqs]
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)
    # whole prompts, as one batch of unequal lengths
    slots = r.admit(3)
    got = r.step(slots, seqs, [list(range(len(s))) for s in seqs]).cpu()
    torch.testing.assert_close(got, torch.cat(want), **tol)
    for s in slots:
        r.release(s)
    # prompts of a part, the rest one token at a time (the state must carry over); slots are reused
    slots = r.admit(3)
    plens = [5, 6, 70]
    r.step(slots, [s[:n] for s, n in zip(seqs, plens)])
    live = [0, 1, 2]
    pos = list(plens)
    while live:
        got = r.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live]).cpu()
        torch.testing.assert_close(got, torch.stack([want[i][pos[i]] for i in live]), **tol)
        for i in live:
            pos[i] += 1
        for i in [i for i in live if pos[i] == len(seqs[i])]:
            r.release(slots[i])
        live = [i for i in live if pos[i] < len(seqs[i])]
    r.cache.check()
