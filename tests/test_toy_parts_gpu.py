"""Parts and architectures defined HERE, in the test, registered and run without a change
to the library: a mixer with fixed-size state of its own (no keys, no values), a run order
that names a layer twice and lets an entry read another entry's cache, a plain pre-norm
arrangement; and, in a second toy, a feed-forward with routing, a position encoding, a norm
and an embedding of their own.  Stepping token by token must give what whole prompts give, and both must give
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
    # prompts fed in pieces of unequal sizes, in steps that others share: one sequence starts while another
    # goes on by 9 tokens and a third by one (the mixer's state is resumed from where the last piece left it;
    # the second attention entry reads the first one's cache over the pieces)
    slots = r.admit(3)
    at = [0, 0, 0]
    plan = [[(0, 11), (2, 40)], [(0, 9), (1, 3), (2, 1)], [(0, 10), (1, 4), (2, 34)]]
    for stepn, entries in enumerate(plan):
        feeds = [seqs[i][at[i]:at[i] + k] for i, k in entries]
        got = r.step([slots[i] for i, _ in entries], feeds, [list(range(len(f))) for f in feeds]).cpu()
        exp = torch.cat([want[i][at[i]:at[i] + k] for i, k in entries])
        torch.testing.assert_close(got, exp, **tol)
        for i, k in entries:
            at[i] += k
    assert at == [30, 7, 75]
    for s in slots:
        r.release(s)
    r.cache.check()


# ---- a second toy: a feed-forward with routing, a position encoding, a norm and an embedding of its
# own, mixed layer by layer with the library's parts ------------------------------------------------

def _register_routed():
    from hos_b200.config.base import LayerCall, LayerSpec, ModelConfig, ModelPlan, PartSpec
    from hos_b200.parts import linear
    from hos_b200.parts.base import FeedForward, Norm, Part, WeightSpec
    from hos_b200.parts.rope import Rotary
    from hos_b200.registry import register_architecture, register_part

    class RoutedFFN(FeedForward):
        """Top-1 of E experts: router logits r = h R^T in 32-bit, expert e = argmax r, output
        softmax(r)[e] * W2_e relu(W1_e h).  Rows are grouped by expert on the host."""

        def __init__(self, spec, rt):
            super().__init__(spec, rt)
            p = spec.params
            self.width, self.inner, self.n_experts = int(p["width"]), int(p["inner"]), int(p["experts"])

        def weight_specs(self):
            w = self.spec.weights
            out = [WeightSpec(w["router"], (self.n_experts, self.width), "matrix", 0.5)]
            for e in range(self.n_experts):
                out.append(WeightSpec(f'{w["experts"]}.{e}.w1', (self.inner, self.width), "matrix", 0.1))
                out.append(WeightSpec(f'{w["experts"]}.{e}.w2', (self.width, self.inner), "matrix", 0.1))
            return out

        def bind(self, tensors):
            w = self.spec.weights
            self.router = tensors[w["router"]].float().contiguous()          # router logits are 32-bit
            self.w1 = [self._matrix(tensors[f'{w["experts"]}.{e}.w1']) for e in range(self.n_experts)]
            self.w2 = [self._matrix(tensors[f'{w["experts"]}.{e}.w2']) for e in range(self.n_experts)]

        def forward(self, h, step):
            r = linear.matmul(h.float(), self.router)                        # [N, E] float32
            gate, choice = torch.softmax(r, -1).max(-1)
            out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
            for e in range(self.n_experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                z = torch.relu(linear.matmul(h[rows].contiguous(), self.w1[e]).float()).to(h.dtype)
                out[rows] = linear.matmul(z, self.w2[e]).float() * gate[rows, None]
            return out.to(h.dtype)

    class ScaledRotary(Rotary):
        """Rotary encoding with all frequencies divided by a factor (position interpolation):
        only the table of inverse frequencies differs, the kernels are the library's."""

        def __init__(self, spec, rt):
            super().__init__(spec, rt)
            self.inv_freq = (self.inv_freq / float(spec.params["factor"])).contiguous()

    class CenteredNorm(Norm):
        """(x - mean) / sqrt(var + eps) * w, written with torch ops: a norm that the fused
        kernels do not know, so the arrangement's default (separate) path runs."""

        def __init__(self, spec, rt):
            super().__init__(spec, rt)
            self.width, self.eps = int(spec.params["width"]), float(spec.params["eps"])

        def weight_specs(self):
            return [WeightSpec(self.spec.weights["weight"], (self.width,), "vector", 0.1)]

        def bind(self, tensors):
            self.w = self._vector32(tensors[self.spec.weights["weight"]])

        def forward(self, x, out=None):
            v = x.float()
            v = v - v.mean(-1, keepdim=True)
            y = (v / torch.sqrt((v * v).mean(-1, keepdim=True) + self.eps) * self.w).to(self.rt.dtype)
            if out is not None:
                out.copy_(y)
                return out
            return y

    class PositionedEmbedding(Part):
        """x = E[token] + P[position]: a learned absolute position, read from the step's positions."""

        def __init__(self, spec, rt):
            super().__init__(spec, rt)
            self.vocab, self.width, self.max_pos = (int(spec.params[k]) for k in ("vocab", "width", "max_pos"))

        def weight_specs(self):
            return [WeightSpec(self.spec.weights["table"], (self.vocab, self.width), "table", 0.5),
                    WeightSpec(self.spec.weights["positions"], (self.max_pos, self.width), "table", 0.5)]

        def bind(self, tensors):
            self.table = tensors[self.spec.weights["table"]].float()
            self.positions = tensors[self.spec.weights["positions"]].float()

        def forward(self, tokens, step=None):
            live = tokens >= 0                                               # padding rows: zeros
            x = self.table[tokens.clamp(min=0).long()] + self.positions[step.token_pos.long()]
            return (x * live[:, None]).contiguous()

    register_part("feed_forward", "toy_routed", RoutedFFN)
    register_part("position", "toy_scaled_rotary", ScaledRotary)
    register_part("norm", "toy_centered", CenteredNorm)
    register_part("embedding", "toy_positioned", PositionedEmbedding)

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        width: int
        vocab: int
        inner: int
        experts: int
        factor: float
        architecture = "ToyRoutedForTests"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["width"], raw["vocab"], raw["inner"], raw["experts"], raw["factor"])

        def to_dict(self):
            return dict(architectures=["ToyRoutedForTests"], width=self.width, vocab=self.vocab, inner=self.inner,
                        experts=self.experts, factor=self.factor, vocab_size=self.vocab)

    def plan(cfg):
        D = cfg.width
        def rms(n):
            return PartSpec("rmsnorm", {"width": D, "eps": 1e-6, "add_one": True}, {"weight": n})
        def centered(n):
            return PartSpec("toy_centered", {"width": D, "eps": 1e-5}, {"weight": n})
        def attn(p, position, window):
            return PartSpec("softmax_attention",
                            {"width": D, "n_heads": 3, "n_kv_heads": 3, "head_dim": 16, "scale": 0.3, "softcap": 20.0,
                             "window": window, "position": position},
                            {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"})
        scaled = PartSpec("toy_scaled_rotary", {"theta": 50.0, "rotary_dim": 16, "style": "rotate_half",
                                                "factor": cfg.factor})
        routed = PartSpec("toy_routed", {"width": D, "inner": cfg.inner, "experts": cfg.experts},
                          {"router": "l0.router", "experts": "l0.experts"})
        dense = PartSpec("gated_mlp", {"width": D, "inner": cfg.inner, "activation": "gelu_tanh"},
                         {"gate": "l1.g", "up": "l1.u", "down": "l1.d"})
        layers = [
            # sandwich arrangement with the library's norm: routed experts behind a window of 9 keys
            LayerSpec("sandwich", attn("l0.", scaled, 9), routed,
                      {"pre_mixer": rms("l0.n1"), "post_mixer": rms("l0.n2"), "pre_ffn": rms("l0.n3"),
                       "post_ffn": rms("l0.n4")}),
            # pre-norm arrangement with the toy norm: no position encoding at all, dense feed-forward
            LayerSpec("prenorm", attn("l1.", PartSpec("none", {}), None), dense,
                      {"pre_mixer": centered("l1.n1"), "pre_ffn": centered("l1.n2")}),
        ]
        return ModelPlan(D, cfg.vocab, 256,
                         PartSpec("toy_positioned", {"vocab": cfg.vocab, "width": D, "max_pos": 256},
                                  {"table": "emb", "positions": "pos"}),
                         layers, [LayerCall(0), LayerCall(1)], centered("final"),
                         PartSpec("linear_head", {"vocab": cfg.vocab, "width": D, "softcap": 0.0}, {"table": "head"}))

    register_architecture("ToyRoutedForTests", RoutedConfig, plan)
    return RoutedConfig


def _plain_routed(w, cfg, tokens):
    """The second toy on one whole sequence, in float32 PyTorch."""
    D, T = cfg.width, len(tokens)
    pos = torch.arange(T, dtype=torch.float32)
    def rms(x, n):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * (1 + w[n])
    def centered(x, n):
        v = x - x.mean(-1, keepdim=True)
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5) * w[n]
    def rope(v):
        inv = 1.0 / torch.pow(torch.tensor(50.0), 2 * torch.arange(8, dtype=torch.float32) / 16) / cfg.factor
        ang = pos[:, None] * inv[None]
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = v[..., :8], v[..., 8:]
        return torch.cat([a * c - b * s, a * s + b * c], -1)
    def attention(h, p, rotate, window):
        q, k, v = ((h @ w[p + n].T).view(T, 3, 16) for n in "qkv")
        if rotate:
            q, k = rope(q), rope(k)
        i = torch.arange(T)
        vis = i[None, :] <= i[:, None]
        if window:
            vis &= i[None, :] > i[:, None] - window
        out = torch.empty(T, 3, 16)
        for hh in range(3):
            s = 20.0 * torch.tanh((q[:, hh] @ k[:, hh].T) * 0.3 / 20.0)
            out[:, hh] = torch.softmax(s.masked_fill(~vis, float("-inf")), -1) @ v[:, hh]
        return out.reshape(T, 48) @ w[p + "o"].T
    def routed(h):
        r = torch.softmax(h @ w["l0.router"].T, -1)
        gate, choice = r.max(-1)
        rows = []
        for t in range(T):
            e = int(choice[t])
            rows.append(gate[t] * (w[f"l0.experts.{e}.w2"] @ torch.relu(w[f"l0.experts.{e}.w1"] @ h[t])))
        return torch.stack(rows)
    def dense(h):
        g = torch.nn.functional.gelu(h @ w["l1.g"].T, approximate="tanh")
        return (g * (h @ w["l1.u"].T)) @ w["l1.d"].T
    x = w["emb"][torch.tensor(tokens)] + w["pos"][:T]
    x = x + rms(attention(rms(x, "l0.n1"), "l0.", True, 9), "l0.n2")
    x = x + rms(routed(rms(x, "l0.n3")), "l0.n4")
    x = x + attention(centered(x, "l1.n1"), "l1.", False, None)
    x = x + dense(centered(x, "l1.n2"))
    return centered(x, "final") @ w["head"].T


def test_toy_architecture_with_routing_and_its_own_position_norm_and_embedding():
    """A feed-forward with routing, a position encoding, a norm and an embedding defined here,
    chosen layer by layer beside the library's parts (sandwich and pre-norm arrangements, a
    window on one layer, no position encoding on the other).  32-bit, so that the router's
    choice is the same on both sides; whole prompts in a batch, then token by token."""
    from hos_b200.engine import Runner
    from hos_b200.model import weight_specs_for
    from hos_b200.weights import RandomSource
    RoutedConfig = _register_routed()
    cfg = RoutedConfig(width=40, vocab=77, inner=56, experts=3, factor=4.0)
    specs = weight_specs_for(cfg)
    assert {"l0.router", "l0.experts.2.w2", "pos", "head", "l1.n1"} <= {s.name for s in specs}
    src = RandomSource(specs, 9)
    r = Runner(cfg, src, dtype="float32", max_tokens=1024)
    assert len(r.cache.groups) == 2                     # a window of 9 keys and all keys: two stores
    w = {n: src.read(n).float() for n in src.names()}
    rng = random.Random(3)
    seqs = [[rng.randrange(77) for _ in range(n)] for n in (40, 3, 21)]
    want = [_plain_routed(w, cfg, s) for s in seqs]
    tol = dict(atol=2e-5, rtol=2e-5)
    slots = r.admit(3)
    got = r.step(slots, seqs, [list(range(len(s))) for s in seqs]).cpu()
    torch.testing.assert_close(got, torch.cat(want), **tol)
    for s in slots:
        r.release(s)
    slots = r.admit(3)
    plens = [12, 1, 20]
    r.step(slots, [s[:n] for s, n in zip(seqs, plens)])
    live, pos = [0, 1, 2], list(plens)
    while live:
        got = r.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live]).cpu()
        torch.testing.assert_close(got, torch.stack([want[i][pos[i]] for i in live]), **tol)
        for i in live:
            pos[i] += 1
        for i in [i for i in live if pos[i] == len(seqs[i])]:
            r.release(slots[i])
        live = [i for i in live if pos[i] < len(seqs[i])]
    r.cache.check()
