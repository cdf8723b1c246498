"""The Zevivik design against its plain statement (``plain_zevivik``): every mechanism alone, then the model
through ``Engine.step`` cut in every way (whole prompts, token by token, portions down to two tokens, unequal
batches, slots and pages used again, blocks of positions and pages crossed while decoding), and greedy generation
through ``Session.generate`` and the command line.  Configurations and weights are made here; where random weights
would hide a fault (a key at a block's edge, a key far back) the inputs are made so that it shows."""
import json

import numpy as np
import pytest
import torch

import plain_zevivik as P
from gpu_util import DEV, TOL, check, scatter_pages
from nncpu_b200 import Engine, GenerateParams, Model, SamplerParams, Session, SessionParams
from nncpu_b200.cache import PAGE
from nncpu_b200.config import config_from_dict
from nncpu_b200.engine.model import parameter_list
from nncpu_b200.kernels import ops
from nncpu_b200.weights import random_tensors, write_safetensors

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


def att(heads, kv, dim, vdim, scale, size=None, rot=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def lat(heads, dim, vdim, rank, scale, mlp=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale},
            "mlp": mlp}


CONFIGS = {
    # odd sizes everywhere: nothing a power of two, value heads wider and narrower than key heads, a block shorter
    # than a page and one longer, a rotation of a part of the head and of all of it, experts with and without a
    # shared one, a layer without a feed-forward, the middle layers run three times
    "P": {"architecture": "Zevivik", "vocab": 301, "width": 88, "norm": {"eps": 3e-6}, "embedding": {"scale": 7.0},
          "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [att(6, 2, 24, 40, 0.3, size=17, rot=(10000.0, 16), mlp=dense(136)),
                     lat(3, 20, 28, 36, 0.25, mlp=moe(5, 2, 40, 1.5, shared=(24, 0.7))),
                     att(4, 4, 16, 12, 0.21, size=70, rot=(500.0, 16), mlp=moe(3, 1, 56, 4.0)),
                     lat(2, 12, 20, 44, 0.4)]},
    # sizes the tensor-core paths take (multiples of 64, head sizes and a latent of 64 and 128); the loop starts at
    # the first layer; a rotation of half a head; blocks of 100 and of 256 positions
    "Q": {"architecture": "Zevivik", "vocab": 512, "width": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
          "loop": {"start": 0, "stop": 2, "times": 2},
          "layers": [att(4, 2, 64, 64, 0.125, size=100, rot=(1000000.0, 64), mlp=dense(512)),
                     lat(4, 32, 64, 128, 0.18, mlp=moe(8, 2, 128, 2.5, shared=(64, 1.0))),
                     att(2, 1, 128, 128, 0.09, size=256, rot=(10000.0, 64), mlp=moe(4, 3, 64, 1.0)),
                     lat(8, 64, 32, 64, 0.125, mlp=dense(256))]},
    # values at the edges and what keeps every fast path out: a width that is no multiple of 8, 32 query heads on one
    # key/value head, blocks of one position (a query sees itself alone) and blocks longer than any sequence here, a
    # rotation of two lanes, no rotation, no mask, every expert chosen, one expert, one latent head with one value
    # lane, a latent of 1 000 lanes, no loop, no embedding scale
    "W": {"architecture": "Zevivik", "vocab": 97, "width": 100, "norm": {"eps": 1e-5},
          "layers": [att(32, 1, 8, 6, 0.5, size=1, rot=(100.0, 2), mlp=moe(4, 4, 20, 0.5, shared=(8, 9.0))),
                     lat(1, 10, 1, 1000, 0.3, mlp=moe(1, 1, 30, 2.0)),
                     att(3, 3, 10, 10, 0.3, size=5000, mlp=dense(36)),
                     att(2, 1, 12, 8, 0.3, rot=(50.0, 12))]},
}


def write_folder(path, cfg_dict, seed, store, sharpen=3.0):
    """A model folder with random weights; the query and key matrices are scaled up so that attention is not
    close to uniform and a key that is wrongly seen or missed changes the logits."""
    config = config_from_dict(cfg_dict)
    tensors = random_tensors(parameter_list(config.model_spec()), seed, store)
    for name in list(tensors):
        if name.endswith((".mix.q", ".mix.k", ".mix.uk")):
            tensors[name] = (tensors[name].float() * sharpen).to(store)
        if name.endswith((".mix.v", ".mix.o", ".mix.dkv", ".up", ".gate", ".down", "embed", "head")):
            tensors[name] = (tensors[name].float() * 3.0).to(store)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config.to_dict()))
    write_safetensors(path / "model.safetensors", tensors, {"format": "pt"})
    return path


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("zevivik")
    return {(name, dtype): write_folder(root / f"{name}_{dtype}", cfg, 11 + i, STORE[dtype])
            for i, (name, cfg) in enumerate(CONFIGS.items()) for dtype in DTYPES}


def toks(cfg, n, seed):
    return np.random.RandomState(seed).randint(0, cfg["vocab"], size=n).tolist()


# -- mechanisms alone -----------------------------------------------------------------------------

def test_gated_activations_on_both_sides_of_their_limits():
    g = torch.Generator().manual_seed(3)
    gu = torch.randn(7, 2 * 33, generator=g) * 3
    gu[0, :4] = torch.tensor([-20.0, 20.0, 1.5, -1.5])
    for kind, limit, want in (("gelu_tanh", 0.0, lambda a, b: P.gelu_tanh(a) * b),
                              ("swish_clamp", 1.5, lambda a, b: np.minimum(a, 1.5) * P.sigmoid(P.GATE_SLOPE * np.minimum(a, 1.5))
                               * (np.clip(b, -1.5, 1.5) + 1.0))):
        out = torch.empty(7, 33, device=DEV)
        ops.gated_act(gu.to(DEV), out, kind, limit)
        a, b = gu[:, :33].double().numpy(), gu[:, 33:].double().numpy()
        check(out, want(a, b), 2e-6, kind)


@pytest.mark.parametrize("m", [1, 8, 16, 17, 40, 64, 100, 256, 300, 600])
@pytest.mark.parametrize("kind,limit", [("gelu_tanh", 0.0), ("swish_clamp", 0.8)])
def test_gated_activations_in_the_epilogue_of_the_tensor_core_products(m, kind, limit):
    """gate and up rows interleaved in blocks of 8, the activation on the 32-bit accumulators, in the few-token
    product and in every tensor-core product, against the product followed by the activation's own kernel."""
    from nncpu_b200.parts import Runtime
    rt = Runtime(DEV, torch.bfloat16)
    g = torch.Generator().manual_seed(m)
    k, inter = 192, 264
    x = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    gate, up = (torch.randn(inter, k, generator=g) * 0.2).bfloat16(), (torch.randn(inter, k, generator=g) * 0.2).bfloat16()
    w = torch.stack([gate.view(-1, 8, k), up.view(-1, 8, k)], dim=1).reshape(-1, k).contiguous().to(DEV)
    got = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    rt.linear(x, w, None, got, epilogue="swiglu", activation=(kind, limit, 0.0))
    a, b = x.double().cpu() @ gate.double().T, x.double().cpu() @ up.double().T
    if kind == "gelu_tanh":
        want = P.gelu_tanh(a.numpy()) * b.numpy()
    else:
        gg = np.minimum(a.numpy(), limit)
        want = gg * P.sigmoid(P.GATE_SLOPE * gg) * (np.clip(b.numpy(), -limit, limit) + 1.0)
    check(got, want, 1e-2, f"{kind} in the epilogue, {m} tokens")
    rt.check_status()


@pytest.mark.parametrize("dim", [88, 100, 256, 1000, 4096])
def test_two_norms_of_the_same_rows_in_one_pass(dim):
    g = torch.Generator().manual_seed(dim)
    x = torch.randn(5, dim, generator=g) * 4
    w1, w2 = 1 + 0.1 * torch.randn(dim, generator=g), 1 + 0.1 * torch.randn(dim, generator=g)
    for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
        y1, y2 = torch.empty(5, dim, dtype=dt, device=DEV), torch.empty(5, dim, dtype=dt, device=DEV)
        ops.rmsnorm_dual(x.to(DEV), w1.to(DEV), 1e-5, w2.to(DEV), 3e-2, y1, y2)
        check(y1, P.rms_norm(x.double().numpy(), w1.double().numpy(), 1e-5), tol, "first norm")
        check(y2, P.rms_norm(x.double().numpy(), w2.double().numpy(), 3e-2), tol, "second norm")


def test_what_a_schedule_adds_to_the_stream():
    g = torch.Generator().manual_seed(5)
    x, rows, vec = torch.randn(6, 52, generator=g), torch.randn(6, 52, generator=g), torch.randn(52, generator=g)
    for r, v in ((rows, vec), (None, vec), (rows, None)):
        got = x.clone().to(DEV)
        ops.stream_add(got, None if r is None else r.to(DEV), None if v is None else v.bfloat16().to(DEV))
        want = x + (0 if r is None else r) + (0 if v is None else v.bfloat16().float())
        check(got, want, 1e-6, "stream add")


@pytest.mark.parametrize("n_experts,top", [(5, 2), (8, 3), (4, 4), (1, 1), (70, 6), (300, 1)])
def test_router_choice_and_weights(n_experts, top):
    """The largest logits in descending order, the lower index on a tie, the softmax over the chosen ones alone."""
    g = torch.Generator().manual_seed(n_experts)
    z = torch.randn(37, n_experts, generator=g) * 2
    if n_experts >= 4:
        z[0, 1] = z[0, 3] = z[0].max() + 1.0       # a tie at the top: the lower index first
        z[1, :] = 0.25                              # all equal
    ids = torch.empty(37, top, dtype=torch.int32, device=DEV)
    ws = torch.empty(37, top, device=DEV)
    ops.moe_route(z.to(DEV), top, ids, ws)
    w = {"m.router": np.eye(n_experts), "m.router.b": np.zeros(n_experts)}
    want_ids, want_ws = P.route(z.double().numpy(), w, "m", top)
    assert ids.cpu().numpy().tolist() == want_ids.tolist()
    check(ws, want_ws, 2e-6, "router weights")
    assert abs(float(ws.sum(dim=1).min()) - 1.0) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,width,ff,E,top", [(1, 88, 40, 5, 2), (9, 100, 30, 3, 1), (40, 256, 128, 8, 3), (3, 64, 7, 2, 2)])
def test_experts_alone(dtype, n, width, ff, E, top):
    dt = STORE[dtype]
    g = torch.Generator().manual_seed(n + ff)
    x = torch.randn(n, width, generator=g).to(dt)
    wg, wu = (torch.randn(E, ff, width, generator=g) * 0.3).to(dt), (torch.randn(E, ff, width, generator=g) * 0.3).to(dt)
    wd = (torch.randn(E, width, ff, generator=g) * 0.3).to(dt)
    z = torch.randn(n, E, generator=g)
    ids, ws = torch.empty(n, top, dtype=torch.int32, device=DEV), torch.empty(n, top, device=DEV)
    ops.moe_route(z.to(DEV), top, ids, ws)
    before = torch.randn(n, width, generator=g)
    out = before.clone().to(DEV)
    act = torch.empty(n * top, ff, dtype=dt, device=DEV)
    ops.moe_experts(x.to(DEV), wg.to(DEV), wu.to(DEV), wd.to(DEV), ids, ws, act, out, "swish_clamp", 1.2)
    w = {}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"] = (t[e].double().numpy() for t in (wg, wu, wd))
    w["m.router"], w["m.router.b"] = np.eye(E), np.zeros(E)
    mlp = {"router": {"top": top}, "expert": {"limit": 1.2}}
    # the router's logits are the rows of z: feed them through an identity router
    want = np.zeros((n, width))
    rid, rws = P.route(z.double().numpy(), w, "m", top)
    for t in range(n):
        for e, a in zip(rid[t], rws[t]):
            want[t] += a * P.expert(x[t:t + 1].double().numpy(), w, f"m.e{e}", 1.2)[0]
    check(out - before.to(DEV), want, 2e-5 if dtype == "float32" else 2e-2, "experts")
    assert mlp["router"]["top"] == top


@pytest.mark.parametrize("n,width,ff,E,top", [(5, 64, 16, 4, 2), (40, 256, 128, 8, 3), (300, 192, 72, 5, 1), (130, 128, 64, 40, 2),
                                              (700, 256, 200, 3, 3), (64, 512, 256, 16, 4)])
def test_experts_as_one_grouped_product_on_the_tensor_cores(n, width, ff, E, top):
    """Token slots sorted by expert, the gate/up product with the activation in its epilogue and the down product as
    grouped products, the choices added up: against the plain experts.  Experts without a token, experts with more
    than a tile of tokens, fewer slots than experts."""
    from nncpu_b200.parts import Runtime
    rt = Runtime(DEV, torch.bfloat16)
    g = torch.Generator().manual_seed(n + ff)
    x = torch.randn(n, width, generator=g).bfloat16()
    wg, wu = (torch.randn(E, ff, width, generator=g) * 0.1).bfloat16(), (torch.randn(E, ff, width, generator=g) * 0.1).bfloat16()
    wd = (torch.randn(E, width, ff, generator=g) * 0.1).bfloat16()
    z = torch.randn(n, E, generator=g)
    if E > 4:
        z[:, 1] = -50.0                      # an expert that nobody is sent to
    ids, ws = torch.empty(n, top, dtype=torch.int32, device=DEV), torch.empty(n, top, device=DEV)
    ops.moe_route(z.to(DEV), top, ids, ws)
    S = n * top
    rows, slots = torch.empty(S, dtype=torch.int32, device=DEV), torch.empty(S, dtype=torch.int32, device=DEV)
    plan = torch.empty(1 + 3 * ops.moe_plan_tiles(S, E), dtype=torch.int32, device=DEV)
    ops.moe_plan(ids, E, rows, slots, plan)
    r = rows.cpu().numpy()
    assert sorted(r.tolist()) == list(range(S)) and (slots.cpu().numpy()[r] == np.arange(S)).all()
    sorted_experts = ids.cpu().numpy().reshape(-1)[slots.cpu().numpy()]
    assert (np.diff(sorted_experts) >= 0).all(), "the rows of an expert follow one another, experts in order"
    xs = torch.empty(S, width, dtype=torch.bfloat16, device=DEV)
    ops.moe_gather(x.to(DEV), slots, top, xs)
    w_mixed = torch.stack([wg.view(E, -1, 8, width), wu.view(E, -1, 8, width)], dim=2).reshape(E, 2 * ff, width).contiguous().to(DEV)
    mid = torch.full((S, ff), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_tc_grouped(xs, w_mixed, mid, plan, E, rt.workspace, "swiglu", ("swish_clamp", 1.2, 0.0))
    y = torch.full((S, width), float("nan"), device=DEV)
    ops.linear_tc_grouped(mid, wd.to(DEV), y, plan, E, rt.workspace)
    before = torch.randn(n, width, generator=g)
    out = before.clone().to(DEV)
    ops.moe_combine(y, rows, ws, out)
    rt.check_status()
    w = {}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"] = (t[e].double().numpy() for t in (wg, wu, wd))
    w["m.router"], w["m.router.b"] = np.eye(E), np.zeros(E)
    rid, rws = P.route(z.double().numpy(), w, "m", top)
    want = np.zeros((n, width))
    for t in range(n):
        for e, a in zip(rid[t], rws[t]):
            want[t] += a * P.expert(x[t:t + 1].double().numpy(), w, f"m.e{e}", 1.2)[0]
    check(out - before.to(DEV), want, 2e-2, "grouped experts")
    # the kernel for few tokens reads the same interleaved layout
    out2 = before.clone().to(DEV)
    act = torch.empty(S, ff, dtype=torch.bfloat16, device=DEV)
    ops.moe_experts(x.to(DEV), w_mixed, None, wd.to(DEV), ids, ws, act, out2, "swish_clamp", 1.2)
    check(out2 - before.to(DEV), want, 2e-2, "experts, interleaved rows")


def test_one_product_per_head_and_the_sigmoid_gate():
    g = torch.Generator().manual_seed(9)
    n, H, K, N = 21, 3, 20, 36
    x = torch.randn(n, 7 + H * K + 5, generator=g)
    w = torch.randn(H, N, K, generator=g)
    gate = torch.randn(n, 11, generator=g)
    out = torch.zeros(n, H * N + 4, device=DEV)
    ops.linear_heads(x.to(DEV), 7, w.to(DEV), out, out_col=4, gate=gate.to(DEV), gate_col=2)
    want = np.zeros((n, H * N + 4))
    for b in range(H):
        y = x[:, 7 + b * K:7 + (b + 1) * K].double().numpy() @ w[b].double().numpy().T
        want[:, 4 + b * N:4 + (b + 1) * N] = y * P.sigmoid(gate[:, 2 + b].double().numpy())[:, None]
    check(out, want, 2e-6, "per-head product")


@pytest.mark.parametrize("n,H,K,N", [(21, 3, 64, 36), (300, 4, 128, 128), (130, 16, 128, 256), (1, 2, 64, 8), (700, 5, 192, 520)])
def test_one_product_per_head_on_the_tensor_cores(n, H, K, N):
    """The same as one grouped product with the heads as groups: a head's columns of the input, its own matrix, its
    columns of the output, the sigmoid gate in the epilogue; bfloat16 and float32 outputs."""
    from nncpu_b200.parts import Runtime
    rt = Runtime(DEV, torch.bfloat16)
    g = torch.Generator().manual_seed(n + N)
    x = torch.randn(n, H * K, generator=g).bfloat16()
    w = (torch.randn(H, N, K, generator=g) * 0.1).bfloat16()
    gate = torch.randn(n, H + 3, generator=g)
    for out_dt, tol in ((torch.bfloat16, 8e-3), (torch.float32, 1e-5)):
        for use_gate in (False, True):
            out = torch.full((n, H * N), float("nan"), dtype=out_dt, device=DEV)
            assert ops.linear_heads_tc_supported(x, 0, w, out)
            ops.linear_heads_tc(x.to(DEV), w.to(DEV), out, rt.workspace, gate=gate.to(DEV) if use_gate else None, gate_col=2)
            rt.check_status()
            want = np.zeros((n, H * N))
            for b in range(H):
                y = x[:, b * K:(b + 1) * K].double().numpy() @ w[b].double().numpy().T
                want[:, b * N:(b + 1) * N] = y * (P.sigmoid(gate[:, 2 + b].double().numpy())[:, None] if use_gate else 1.0)
            check(out, want, tol, f"per-head product on the tensor cores, {out_dt}, gate {use_gate}")


def test_rotation_of_a_part_of_the_head():
    """The first ``dims`` lanes turn, lane i with lane i + dims/2; the others pass."""
    nh, nkv, hd, dims, base = 3, 1, 24, 10, 777.0
    pos = [0, 1, 5, 63, 64, 900]
    n = len(pos)
    g = torch.Generator().manual_seed(2)
    qkv = torch.randn(n, (nh + 2 * nkv) * hd, generator=g)
    inv = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32, device=DEV)
    cs = torch.empty(n, dims // 2, 2, device=DEV)
    tp = torch.tensor(pos, dtype=torch.int32, device=DEV)
    ops.rope_table(tp, inv, cs)
    kp = torch.zeros(16, nkv, PAGE, hd, device=DEV)
    vp = torch.zeros(16, nkv, PAGE, hd, device=DEV)
    table = torch.arange(16, dtype=torch.int32, device=DEV).view(1, 16)
    q_out = torch.empty(n, nh * hd, device=DEV)
    ops.qk_norm_rope_append(qkv.to(DEV), None, None, 0.0, cs, torch.zeros(n, dtype=torch.int32, device=DEV), tp, table, kp, vp,
                            q_out, nh, nkv, hd)
    want_q = P.rotate(qkv[:, :nh * hd].double().numpy().reshape(n, nh, hd), pos, base, dims)
    check(q_out.view(n, nh, hd), want_q, 2e-5, "rotated queries")      # 32-bit angles at position 900
    assert torch.equal(q_out.view(n, nh, hd)[:, :, dims:].cpu(), qkv[:, :nh * hd].view(n, nh, hd)[:, :, dims:])
    want_k = P.rotate(qkv[:, nh * hd:(nh + nkv) * hd].double().numpy().reshape(n, nkv, hd), pos, base, dims)
    got_k = torch.stack([kp[p // PAGE, :, p % PAGE] for p in pos])
    check(got_k, want_k, 2e-5, "rotated keys in their pages")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,vd,size", [(6, 2, 24, 40, 17), (4, 4, 16, 12, 70), (5, 1, 32, 32, 1), (4, 2, 64, 64, 100),
                                               (2, 1, 128, 128, 64), (3, 3, 8, 8, 1000)])
def test_attention_inside_blocks_of_positions_alone(dtype, nh, nkv, hd, vd, size):
    """Queries at the end of two sequences (a prompt's portion of 9 tokens, one decoded token) over shuffled pages."""
    dt = STORE[dtype]
    lens = [150, 67]
    g = torch.Generator().manual_seed(hd + vd)
    kp, _, table, ks, _ = scatter_pages(9, nkv, hd, lens, dt, seed=1)
    _, vp, _, _, vs = scatter_pages(9, nkv, vd, lens, dt, seed=1)
    new = [9, 1]
    q = [torch.randn(n, nh, hd, generator=g).to(dt) for n in new]
    tok_seq = torch.tensor([0] * 9 + [1], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(list(range(lens[0] - 9, lens[0])) + [lens[1] - 1], dtype=torch.int32, device=DEV)
    out = torch.empty(10, nh * vd, dtype=dt, device=DEV)
    ops.attention(torch.cat(q).view(10, -1).to(DEV), kp, vp, table, tok_seq, tok_pos, out, nh, nkv, hd, 0.2,
                  ops.key_span(chunk=size), vd)
    want = torch.cat([torch.from_numpy(P.masked_attention(
        q[b].double().numpy(), ks[b].double().numpy(), vs[b].double().numpy(), range(lens[b] - new[b], lens[b]), 0.2, size))
        for b in range(2)]).view(10, -1)
    check(out, want, 2e-5 if dtype == "float32" else 2e-2, "attention inside blocks")


@pytest.mark.parametrize("nh,nkv,hd,size", [(4, 2, 64, 100), (2, 1, 128, 64), (8, 2, 64, 56), (16, 1, 64, 0), (12, 4, 128, 200),
                                            (6, 2, 64, 30), (3, 1, 128, 129), (5, 5, 64, 70), (1, 1, 64, 3), (2, 2, 128, 1)])
def test_attention_inside_blocks_on_the_tensor_core_kernels(nh, nkv, hd, size):
    """The bfloat16 kernels for prompts and for decode steps: three sequences (a portion of 9 tokens, a whole prompt
    of 67, a portion of 130 that crosses pages and blocks), then one token each, with the keys in one split and in two."""
    lens, new = [150, 67, 300], [9, 67, 130]
    g = torch.Generator().manual_seed(nh + hd)
    kp, vp, table, ks, vs = scatter_pages(12, nkv, hd, lens, torch.bfloat16, seed=3)
    q = [torch.randn(n, nh, hd, generator=g).bfloat16() for n in new]
    n = sum(new)
    span = ops.key_span(chunk=size)
    cu = torch.tensor(np.cumsum([0] + new), dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([p for b in range(3) for p in range(lens[b] - new[b], lens[b])], dtype=torch.int32, device=DEV)
    out = torch.empty(n, nh * hd, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill_mma(torch.cat(q).view(n, -1).to(DEV), kp, vp, table, cu, tok_pos, out, 3, nh, nkv, hd, 0.2, span)
    want = torch.cat([torch.from_numpy(P.masked_attention(
        q[b].double().numpy(), ks[b].double().numpy(), vs[b].double().numpy(), range(lens[b] - new[b], lens[b]), 0.2, size))
        for b in range(3)]).view(n, -1)
    check(out, want, 2e-2, "prompt kernel")
    if ops.attention_prefill_tc_supported(nh, nkv, hd):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out_tc = torch.empty_like(out)
        ops.attention_prefill_tc(torch.cat(q).view(n, -1).to(DEV), kp, vp, table, cu, tok_pos, out_tc, status, 3, nh, nkv, hd,
                                 0.2, span)
        assert int(status.item()) == 0
        check(out_tc, want, 2e-2, "tcgen05 prompt kernel")
    last = torch.stack([q[b][-1] for b in range(3)]).view(3, -1).to(DEV)
    seq = torch.arange(3, dtype=torch.int32, device=DEV)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    want = torch.stack([want[int(cu[b + 1]) - 1] for b in range(3)])
    for n_splits in (1, 2):
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(ops.attention_decode_scratch_floats(3, nh, nkv, hd, n_splits), device=DEV)
        got = torch.empty(3, nh * hd, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode_mma(last, kp, vp, table, seq, pos, got, scratch, nh, nkv, hd, 0.2, span, n_splits)
        check(got, want, 2e-2, f"decode kernel, {n_splits} splits")


@pytest.mark.parametrize("size", [1, 5, 64, 65, 100, 130])
def test_block_edge_one_key_inside_one_outside(size):
    """One key's score stands out (its query and key are scaled up).  As the first key of the query's block it is
    seen and the output is its value; as the last key of the block before it is not, and the output must not know it.
    Queries at a block's first and last position and in its middle, with the key on the far side of a page border too;
    in the 32-bit kernel and, at a head size they take, in the bfloat16 kernels for decode steps and portions."""
    nkv, n = 1, 300
    for nh, hd, fast in ((2, 16, False), (2, 64, True)):
        for query in sorted({n - 1, (n - 1) // size * size, min(n - 1, 2 * size + size // 2), min(n - 1, 3 * size - 1)}):
            start = query // size * size
            for inside in (True, False):
                far = start if inside else start - 1
                if far < 0:
                    continue
                dt = torch.bfloat16 if fast else torch.float32
                kp, vp, table, ks, vs = scatter_pages(6, nkv, hd, [n], dt, seed=2)
                q = (torch.randn(1, nh, hd, generator=torch.Generator().manual_seed(size)) * 0.1)
                q[0, :, 3] = 40.0
                page, row = int(table[0, far // PAGE]), far % PAGE
                kp[page, 0, row] = 0
                kp[page, 0, row, 3] = 40.0
                ks[0][far] = kp[page, 0, row].float().cpu()
                args = (table, torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([query], dtype=torch.int32, device=DEV))
                want = P.masked_attention(q.to(dt).double().numpy(), ks[0][:query + 1].double().numpy(),
                                          vs[0][:query + 1].double().numpy(), [query], 1.0, size)
                outs = {}
                out = torch.empty(1, nh * hd, dtype=dt, device=DEV)
                ops.attention(q.view(1, -1).to(dt).to(DEV), kp, vp, *args, out, nh, nkv, hd, 1.0, ops.key_span(chunk=size))
                outs["32-bit kernel"] = out
                if fast:
                    out = torch.empty(1, nh * hd, dtype=dt, device=DEV)
                    ops.attention_decode_mma(q.view(1, -1).to(dt).to(DEV), kp, vp, *args, out, None, nh, nkv, hd, 1.0,
                                             ops.key_span(chunk=size), 1)
                    outs["decode kernel"] = out
                    out = torch.empty(1, nh * hd, dtype=dt, device=DEV)
                    cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
                    ops.attention_prefill_mma(q.view(1, -1).to(dt).to(DEV), kp, vp, table, cu, args[2], out, 1, nh, nkv, hd, 1.0,
                                              ops.key_span(chunk=size))
                    outs["portion kernel"] = out
                for what, out in outs.items():
                    check(out.view(1, nh, hd), want, 2e-2 if fast else 1e-5, f"{what}, blocks of {size}, query {query}")
                    hit = float((out.view(nh, hd)[0].float().cpu() - vs[0][far, 0]).abs().max())
                    assert (hit < 2e-2) == inside, f"{what}, blocks of {size}, query {query}: the key at {far} is {'missed' if inside else 'seen'}"


# -- the model ------------------------------------------------------------------------------------

def close(got, want, dtype, what):
    """Logits against the plain model's.  float32: the largest difference within 1e-4 of the largest logit.
    bfloat16: rounding of the activations to 8 bits of mantissa is the design's own noise, so the measure is the
    root mean square of the differences over all the rows given, held to 4 % of the logits' own; a fault of the cache
    or of a block's edge moves far more than that with these weights, and the float32 runs hold the same code to
    1e-4.  Rows are judged together, not one by one: where two router logits are closer than the noise, a bfloat16
    run may send a token to another expert than the plain model does, which moves that one row by a tenth or so."""
    if dtype == "float32":
        return check(got, want, TOL[dtype], what)
    g = got.detach().double().cpu().numpy()
    w = np.asarray(want, dtype=np.float64).reshape(g.shape)
    assert np.isfinite(g).all(), f"{what}: NaN or infinity"
    rms = float(np.sqrt(np.mean((g - w) ** 2)) / np.sqrt(np.mean(w ** 2)))
    assert rms <= 4e-2, f"{what}: root mean square of the differences {rms:.3e} of the logits' own"
    check(got, want, 0.25, what)


class Rows:
    """Rows of logits that arrive one step at a time: float32 rows are judged as they come, bfloat16 rows together
    at the end (see ``close``)."""

    def __init__(self, dtype, what):
        self.dtype, self.what, self.got, self.want = dtype, what, [], []

    def add(self, got, want, where=""):
        if self.dtype == "float32":
            return close(got, want, self.dtype, f"{self.what} {where}")
        self.got.append(got.detach().float().reshape(-1).clone())
        self.want.append(np.asarray(want, dtype=np.float64).reshape(-1))

    def done(self):
        if self.got:
            close(torch.stack(self.got), np.stack(self.want), self.dtype, self.what)


def plain_logits(folder, tokens):
    cfg, w = P.load(folder)
    return P.forward(cfg, w, tokens)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_every_position(folders, name, dtype):
    cfg = CONFIGS[name]
    t = toks(cfg, 150, 1)
    want = plain_logits(folders[name, dtype], t)
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=256)
    got = engine.step([engine.alloc_slot()], [t], [list(range(150))])
    close(got, want, dtype, f"{name} whole prompt")
    if dtype == "float32":         # the first tokens of a sequence, one by one in the sharper arithmetic
        for i in range(4):
            close(got[i], want[i], dtype, f"{name} token {i}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_every_layer_run_against_the_plain_model(folders, dtype):
    """The stream after every run of a layer (the looped ones every time), float32 and bfloat16."""
    name = "P"
    t = toks(CONFIGS[name], 40, 4)
    cfg, w = P.load(folders[name, dtype])
    trace = []
    P.forward(cfg, w, t, trace)
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64, use_graphs=False)
    caught = []
    for b in set(model.blocks):
        def wrapped(ctx, residual, caches, _o=b.forward):
            _o(ctx, residual, caches)
            caught.append(residual.detach().clone())
        b.forward = wrapped
    engine.step([engine.alloc_slot()], [t], [[39]])
    assert len(caught) == len(trace) == 1 + 2 * 3 + 1
    for r, (got, want) in enumerate(zip(caught, trace)):
        check(got, want, 1e-5 if dtype == "float32" else 3e-2, f"stream after layer run {r}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_token_by_token_against_the_whole(folders, name, dtype):
    """The same 200 tokens: whole; in portions of 2, 3, 64, 1, 65, ... tokens; a prompt of 40 and then one token a
    step for 160 steps (across blocks and page borders).  All against the plain model; in float32 the three
    runs agree with one another far below the tolerance."""
    cfg = CONFIGS[name]
    t = toks(cfg, 200, 2)
    want = plain_logits(folders[name, dtype], t)
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 12)
    s = engine.alloc_slot()
    whole = engine.step([s], [t], [list(range(200))]).clone()
    close(whole, want, dtype, "whole")
    s2 = engine.alloc_slot()
    rows, at, sizes, i = [], 0, [2, 3, 64, 1, 65, 2, 7], 0
    while at < 200:
        n = min(sizes[i % len(sizes)], 200 - at)
        rows.append(engine.step([s2], [t[at:at + n]], [list(range(n))]).clone())
        at += n
        i += 1
    portions = torch.cat(rows)
    close(portions, want, dtype, "portions")
    engine.free_slot(s)
    s3 = engine.alloc_slot()                 # the slot and pages that the whole run used
    engine.step([s3], [t[:40]], [[]])
    rows = [engine.step([s3], [[t[i]]]).clone() for i in range(40, 200)]
    decoded = torch.cat(rows)
    close(decoded, want[40:], dtype, "token by token")
    s4 = engine.alloc_slot()                 # portions that want their last place only: the captured prompt steps
    at, last = 0, []
    for n in (5, 2, 33, 2, 100, 58):
        last.append(engine.step([s4], [t[at:at + n]]).clone())
        at += n
    close(torch.cat(last), want[[4, 6, 39, 41, 141, 199]], dtype, "portions through captured steps")
    if dtype == "float32":
        check(portions, whole, 2e-5, "portions against the whole")
        check(decoded, whole[40:], 2e-5, "token by token against the whole")
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batch_then_decoding_together_on_reused_slots(folders, name, dtype):
    """Four prompts of 1, 33, 130 and 64 tokens in one step, then one token each per step; the short ones end
    early and give their slots and pages back; a newcomer takes them while the others go on."""
    cfg = CONFIGS[name]
    lens, tails = [1, 33, 130, 64], [3, 10, 24, 24]
    seqs = [toks(cfg, n + k, 10 + i) for i, (n, k) in enumerate(zip(lens, tails))]
    want = [plain_logits(folders[name, dtype], t) for t in seqs]
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 8)
    slots = [engine.alloc_slot() for _ in seqs]
    out = engine.step(slots, [t[:n] for t, n in zip(seqs, lens)], [[n - 1] for n in lens])
    rows = [Rows(dtype, f"sequence {b}") for b in range(4)]
    for b in range(4):
        rows[b].add(out[b], want[b][lens[b] - 1], "prompt")
    live = list(range(4))
    newcomer = toks(cfg, 90, 99)
    want_new = plain_logits(folders[name, dtype], newcomer)
    for step in range(24):
        live = [b for b in live if step < tails[b]]
        out = engine.step([slots[b] for b in live], [[seqs[b][lens[b] + step]] for b in live])
        for i, b in enumerate(live):
            rows[b].add(out[i], want[b][lens[b] + step], f"decoded token {step}")
        for b in list(range(4)):
            if step + 1 == tails[b] and b in live and tails[b] < 24:
                engine.free_slot(slots[b])
        if step == 11:                      # both short sequences are gone: their slots and pages are used again
            s = engine.alloc_slot()
            got = engine.step([s], [newcomer], [[0, 1, 63, 64, 89]])
            close(got, want_new[[0, 1, 63, 64, 89]], dtype, "a newcomer on used slots")
            engine.free_slot(s)
    for r in rows:
        r.done()
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_across_blocks_and_pages(folders, dtype):
    """420 decoded tokens after a prompt of 150: blocks of 100 and 256 positions and pages pass by, the pages of
    blocks that are over go back to the pool, and a latent layer's keys go back 570 positions."""
    cfg = CONFIGS["Q"]
    n = 570
    t = toks(cfg, n, 5)
    want = plain_logits(folders["Q", dtype], t)
    model = Model.load(folders["Q", dtype], dtype=dtype)
    engine = Engine(model, max_tokens=640)
    s = engine.alloc_slot()
    engine.step([s], [t[:150]], [[]])
    rows = Rows(dtype, "long decoding")
    for i in range(150, n):
        out = engine.step([s], [[t[i]]])
        if i % 7 == 0 or i % 100 in (99, 0, 1) or i % 256 in (255, 0, 1) or i > n - 10:
            rows.add(out[0], want[i], f"decoded position {i}")
    rows.done()
    held = sorted(g.pool.n_held for g in engine.cache.groups)
    assert held[0] <= 2 and held[-1] == 9, held       # block groups keep their current block; the latent keeps all
    engine.cache.check()


def test_long_prompt_through_the_fused_projection_epilogue_and_the_grouped_experts(tmp_path):
    """Head size 128, whole heads rotated, 600 tokens in one step: the q/k/v product's epilogue rotates and appends, the
    tcgen05 prompt kernel masks by blocks of 200, the experts run as a grouped product; then ten tokens one by one
    (attention from the projections).  bfloat16 against the plain model, and against the same model run in float32."""
    cfg = {"architecture": "Zevivik", "vocab": 300, "width": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "loop": {"start": 0, "stop": 1, "times": 2},
           "layers": [att(4, 2, 128, 128, 0.09, size=200, rot=(1000000.0, 128), mlp=moe(4, 2, 64, 2.0, shared=(128, 1.0))),
                      lat(4, 64, 64, 128, 0.125, mlp=dense(256))]}
    folder = write_folder(tmp_path / "m", cfg, 5, torch.bfloat16, sharpen=2.0)
    t = toks(cfg, 610, 3)
    want = plain_logits(folder, t)
    rows = list(range(0, 600, 7)) + [198, 199, 200, 201, 399, 400, 599]
    for dtype in ("bfloat16", "float32"):
        model = Model.load(folder, dtype=dtype)
        engine = Engine(model, max_tokens=64 * 11)
        s = engine.alloc_slot()
        close(engine.step([s], [t[:600]], [rows]), want[rows], dtype, f"{dtype}: a prompt of 600 tokens")
        out = torch.cat([engine.step([s], [[t[i]]]).clone() for i in range(600, 610)])
        close(out, want[600:], dtype, f"{dtype}: ten tokens after it")
        model.rt.check_status()


def test_a_key_far_back_in_a_latent_layer(tmp_path):
    """One latent layer with queries and keys so sharp that single keys take most of a row's weight, most of them far
    back and across pages (560 positions, every key visible): the logits must follow the plain model as a prompt and
    token by token."""
    cfg = {"architecture": "Zevivik", "vocab": 64, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": [lat(2, 16, 24, 40, 1.0, mlp=dense(64))]}
    folder = write_folder(tmp_path / "m", cfg, 3, torch.float32, sharpen=12.0)
    t = toks(cfg, 560, 8)
    want = plain_logits(folder, t)
    model = Model.load(folder, dtype="float32")
    engine = Engine(model, max_tokens=1280)
    s = engine.alloc_slot()
    got = engine.step([s], [t], [[20, 529, 530, 559]])
    check(got, want[[20, 529, 530, 559]], 1e-4, "a prompt with a far key")
    s2 = engine.alloc_slot()
    engine.step([s2], [t[:500]], [[]])
    for i in range(500, 535):
        out = engine.step([s2], [[t[i]]])
    check(out[0], want[534], 1e-4, "decoded past a far key")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_session(folders, name):
    """``Session.generate`` (scheduler, batches, captured decode steps) against greedy decoding of the plain model."""
    cfg = CONFIGS[name]
    folder = folders[name, "float32"]
    pcfg, w = P.load(folder)
    prompts = [toks(cfg, 70, 21), toks(cfg, 3, 22), toks(cfg, 129, 23)]
    want = [P.greedy(pcfg, w, p, 8) for p in prompts]
    model = Model.load(folder, dtype="float32")
    session = Session(model, SessionParams(n_ctx=256, seed=1, max_batch=2))
    res = session.generate(prompts, GenerateParams(8, SamplerParams.greedy()), stop_token_ids=())
    assert [r.tokens for r in res] == want
    # the same in bfloat16: the length of every reply (tokens may part ways by rounding)
    model = Model.load(folders[name, "bfloat16"], dtype="bfloat16")
    session = Session(model, SessionParams(n_ctx=256, seed=1, max_batch=3))
    res = session.generate(prompts, GenerateParams(4, SamplerParams.greedy()), stop_token_ids=())
    assert all(len(r.tokens) == 4 for r in res)


def test_command_line_random_weights_info_and_generation(tmp_path):
    """The command line's modes on this design: a folder with random weights from a configuration file, its --info,
    the greedy token harness against the plain model, and a sampled continuation (device-side sampling chain)."""
    import io
    from nncpu_b200.cli import parse_options, run_gen, run_generate, run_info, run_random_weights

    def run(fn, argv):
        out = io.StringIO()
        assert fn(parse_options(argv), out) == 0
        return out.getvalue()

    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(CONFIGS["P"]))
    run(run_random_weights, ["--random-weights", str(cfg), "5", str(tmp_path / "m"), "--fp32"])
    info = json.loads(run(run_info, ["--info", str(tmp_path / "m")]))
    assert info["config"]["architecture"] == "Zevivik" and info["parameters"] > 0
    prompt = toks(CONFIGS["P"], 40, 3)
    got = [int(t) for t in run(run_gen, ["--gen", str(tmp_path / "m"), " ".join(map(str, prompt)), "6", "--fp32"]).splitlines()[0].split()]
    pcfg, w = P.load(tmp_path / "m")
    assert got == P.greedy(pcfg, w, prompt, 6)
    out = run(run_generate, ["-m", str(tmp_path / "m"), "--tokens", " ".join(map(str, prompt)), "-n", "6", "--temp", "0.8",
                             "--top-k", "20", "-s", "4", "-b", "3"]).split()
    assert len(out) >= 6 and all(0 <= int(t) < CONFIGS["P"]["vocab"] for t in out[:6])
