"""Each kind of part alone, built from a PartSpec through the registry, against the plain
implementation's function for that part."""
import math

import pytest
import torch

from plain import gemma2_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOLS = {"float32": dict(atol=1e-5, rtol=1e-5), "bfloat16": dict(atol=2e-2, rtol=2e-2)}


def close(a, b, dtype):
    torch.testing.assert_close(a.float().cpu(), b.float().cpu(), **TOLS[dtype])


def rt(dtype):
    from hos_b200.parts.base import Runtime
    return Runtime(torch.device(DEV), DT[dtype])


def rand_weights(part, seed=0):
    from hos_b200.weights import RandomSource
    src = RandomSource(part.weight_specs(), seed)
    t = {n: src.read(n).to(DEV) for n in src.names()}
    for s in part.weight_specs():
        if s.name not in t and s.fallback:
            t[s.name] = t[s.fallback]
    return t


def step_for(lens, starts, slots, vocab=1000):
    from hos_b200.engine.batch import build_step
    toks = [[1] * n for n in lens]
    return build_step(toks, starts, slots, torch.device(DEV), vocab)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from hos_b200.config import PartSpec
    from hos_b200.registry import part_impl
    spec = PartSpec("rmsnorm", {"width": 72, "eps": 1e-4, "add_one": True}, {"weight": "n.w"})
    n = part_impl("norm", "rmsnorm")(spec, rt(dtype))
    w = rand_weights(n)
    n.bind(w)
    x = torch.randn(9, 72, device=DEV)
    close(n.forward(x), P.rmsnorm(x.cpu(), w["n.w"].float().cpu(), 1e-4).to(DT[dtype]), dtype)
    y = torch.randn(9, 72, device=DEV).to(DT[dtype])
    x2 = x.clone()
    h = n.add_to(y, x2, then=n)
    want_x = x.cpu() + P.rmsnorm(y.float().cpu(), w["n.w"].float().cpu(), 1e-4)
    close(x2, want_x, "float32")
    close(h, P.rmsnorm(want_x, w["n.w"].float().cpu(), 1e-4).to(DT[dtype]), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    from hos_b200.config import PartSpec
    from hos_b200.registry import part_impl
    V, D = 331, 88
    e = part_impl("embedding", "scaled_embedding")(
        PartSpec("scaled_embedding", {"vocab": V, "width": D, "scale": math.sqrt(D)}, {"table": "emb"}), rt(dtype))
    w = rand_weights(e)
    e.bind(w)
    toks = [0, 330, 17]
    x = e.forward(torch.tensor(toks, dtype=torch.int32, device=DEV))
    assert x.dtype == torch.float32
    close(x, P.embed(w["emb"].cpu(), toks, D), "float32")
    hd = part_impl("head", "linear_head")(
        PartSpec("linear_head", {"vocab": V, "width": D, "softcap": 2.0}, {"table": "head", "tied_to": "emb"}),
        rt(dtype))
    hd.bind({"head": w["emb"]})
    h = (torch.randn(5, D, device=DEV) * 4).to(DT[dtype])
    got = hd.forward(h)
    assert got.dtype == torch.float32 and got.shape == (5, V)
    close(got, P.softcap(P.linear(h.float().cpu(), w["emb"].cpu()), 2.0), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_gated_mlp_part(dtype, act):
    from hos_b200.config import PartSpec
    from hos_b200.registry import part_impl
    spec = PartSpec("gated_mlp", {"width": 72, "inner": 200, "activation": act},
                    {"gate": "g", "up": "u", "down": "d"})
    f = part_impl("feed_forward", "gated_mlp")(spec, rt(dtype))
    w = rand_weights(f)
    f.bind(w)
    h = torch.randn(11, 72, device=DEV).to(DT[dtype])
    got = f.forward(h)
    hc = h.float().cpu()
    g, u = P.linear(hc, w["g"].cpu()), P.linear(hc, w["u"].cpu())
    a = P.gelu_tanh(g) if act == "gelu_tanh" else g / (1 + torch.exp(-g))
    close(got, P.linear(a * u, w["d"].cpu()).to(DT[dtype]), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_prompt_then_decode(dtype, window):
    """The mixer alone with a cache of its own: two prompts of unequal length in one step,
    then single tokens, against the plain attention block on the whole sequences."""
    from hos_b200.cache import CacheManager
    from hos_b200.config import PartSpec
    from hos_b200.registry import part_impl
    D, nh, nkv, hd = 72, 6, 2, 16
    pos_spec = PartSpec("rotary", {"theta": 777.0, "rotary_dim": hd, "style": "rotate_half"})
    spec = PartSpec("softmax_attention",
                    {"width": D, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "scale": 0.31,
                     "softcap": 9.0, "window": window, "position": pos_spec},
                    {"q": "q", "k": "k", "v": "v", "o": "o"})
    m = part_impl("mixer", "softmax_attention")(spec, rt(dtype))
    w = rand_weights(m)
    m.bind(w)
    cache = CacheManager([m.kv_need()], [None], [[]], 1024, 256, DT[dtype], torch.device(DEV))
    lens, total = [70, 9], [90, 30]
    hs = [torch.randn(t, D).to(DT[dtype]).float() for t in total]
    # the plain attention block includes the input norm: undo it by feeding rows that the norm leaves as they are
    def plain_block(hrows):
        T = hrows.shape[0]
        q = P.linear(hrows, w["q"].cpu()).view(T, nh, hd)
        k = P.linear(hrows, w["k"].cpu()).view(T, nkv, hd)
        v = P.linear(hrows, w["v"].cpu()).view(T, nkv, hd)
        q = P.rope_rotate_half(q, torch.arange(T), hd, 777.0)
        k = P.rope_rotate_half(k, torch.arange(T), hd, 777.0)
        return P.linear(P.attention(q, k, v, 0.31, 9.0, window).reshape(T, -1), w["o"].cpu())
    want = [plain_block(h) for h in hs]
    slots = cache.admit([0, 0])
    for s, n in zip(slots, lens):
        cache.extend(s, n)
    cache.flush()
    step = step_for(lens, [0, 0], slots)
    h_in = torch.cat([hs[0][:70], hs[1][:9]]).to(DEV).to(DT[dtype])
    got = m.forward(h_in, step, cache.stores[0])
    close(got, torch.cat([want[0][:70], want[1][:9]]).to(DT[dtype]), dtype)
    for t in range(20):
        for s, n in zip(slots, lens):
            cache.extend(s, n + t + 1)
        cache.flush()
        step = step_for([1, 1], [lens[0] + t, lens[1] + t], slots)
        h_in = torch.stack([hs[0][70 + t], hs[1][9 + t]]).to(DEV).to(DT[dtype])
        got = m.forward(h_in, step, cache.stores[0])
        close(got, torch.stack([want[0][70 + t], want[1][9 + t]]).to(DT[dtype]), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("arrangement", ["sandwich", "prenorm"])
def test_layer_arrangements(dtype, arrangement):
    from hos_b200.cache import CacheManager
    from hos_b200.config import LayerSpec, PartSpec
    from hos_b200.registry import part_impl
    D, nh, nkv, hd, F = 64, 4, 4, 16, 96
    def norm(name):
        return PartSpec("rmsnorm", {"width": D, "eps": 1e-6, "add_one": True}, {"weight": name})
    mixer = PartSpec("softmax_attention",
                     {"width": D, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "scale": 0.25, "softcap": 0.0,
                      "window": None, "position": PartSpec("rotary", {"theta": 1e4, "rotary_dim": hd})},
                     {"q": "q", "k": "k", "v": "v", "o": "o"})
    ffn = PartSpec("gated_mlp", {"width": D, "inner": F, "activation": "gelu_tanh"},
                   {"gate": "g", "up": "u", "down": "d"})
    roles = ["pre_mixer", "post_mixer", "pre_ffn", "post_ffn"] if arrangement == "sandwich" else ["pre_mixer", "pre_ffn"]
    layer = part_impl("arrangement", arrangement)(LayerSpec(arrangement, mixer, ffn, {r: norm(r) for r in roles}),
                                                  rt(dtype))
    w = {}
    for p in layer.parts():
        w.update(rand_weights(p, seed=3))
    for p in layer.parts():
        p.bind(w)
    cw = {k: v.float().cpu() for k, v in w.items()}
    T = 21
    x0 = torch.randn(T, D)
    cache = CacheManager([layer.mixer.kv_need()], [None], [[]], 256, 128, DT[dtype], torch.device(DEV))
    slot = cache.admit([0])[0]
    cache.extend(slot, T)
    cache.flush()
    x = x0.to(DEV).clone()
    layer.forward(x, step_for([T], [0], [slot]), cache.stores[0])
    # plain
    def attn(hrows):
        q = P.linear(hrows, cw["q"]).view(T, nh, hd)
        k = P.linear(hrows, cw["k"]).view(T, nkv, hd)
        v = P.linear(hrows, cw["v"]).view(T, nkv, hd)
        q, k = (P.rope_rotate_half(t, torch.arange(T), hd, 1e4) for t in (q, k))
        return P.linear(P.attention(q, k, v, 0.25, 0.0, None).reshape(T, -1), cw["o"])
    def mlp(hrows):
        return P.linear(P.gelu_tanh(P.linear(hrows, cw["g"])) * P.linear(hrows, cw["u"]), cw["d"])
    xr = x0.clone()
    a = attn(P.rmsnorm(xr, cw["pre_mixer"], 1e-6))
    xr = xr + (P.rmsnorm(a, cw["post_mixer"], 1e-6) if arrangement == "sandwich" else a)
    f = mlp(P.rmsnorm(xr, cw["pre_ffn"], 1e-6))
    xr = xr + (P.rmsnorm(f, cw["post_ffn"], 1e-6) if arrangement == "sandwich" else f)
    assert x.dtype == torch.float32
    close(x, xr, dtype)
