"""The Romepel design against its plain statement (``plain_romepel``): every mechanism alone, then the model
through ``Engine.step`` cut in every way (whole prompts, token by token, portions down to two tokens, unequal
batches, slots and pages used again, windows and pages crossed while decoding), and greedy generation through
``Session.generate``.  Configurations and weights are made here; where random weights would hide a fault (a key
at a window's edge, a token far back in a recurrent state) the inputs are made so that it shows."""
import json

import numpy as np
import pytest
import torch

import plain_romepel as P
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


def att(heads, kv, dim, vdim, scale, window=None, q_temp=None, ff=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def gla(heads, dim, vdim, tau, rank, ff=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


CONFIGS = {
    # odd sizes everywhere: nothing a power of two, value heads wider and narrower than key heads, a window
    # shorter than a page and one longer, a layer without a window or a temperature, a feed-forward on a gla layer
    "R": {"architecture": "Romepel", "vocab": 301, "width": 88, "max_positions": 700, "norm": {"eps": 3e-6},
          "logit_softcap": 9.0,
          "layers": [att(6, 2, 24, 40, 0.3, window=17, q_temp=(0.7, 5), ff=136),
                     gla(3, 20, 48, 7.0, 5, ff=72),
                     att(4, 4, 16, 12, 0.21),
                     gla(2, 40, 24, 3.0, 12),
                     att(5, 1, 32, 32, 0.11, window=70, q_temp=(0.2, 64), ff=64)]},
    # sizes the tensor-core paths take (multiples of 64, head sizes 64 and 128), one layer of each kind first
    # the other way round, values that a model may make equal or 1: one head, one key/value head, rank 8
    "S": {"architecture": "Romepel", "vocab": 512, "width": 256, "max_positions": 1024, "norm": {"eps": 1e-5},
          "layers": [gla(1, 64, 128, 24.0, 8),
                     att(4, 2, 64, 64, 0.125, window=100, q_temp=(0.4, 32), ff=512),
                     att(2, 1, 128, 128, 0.09, window=256, ff=256),
                     gla(4, 128, 64, 12.0, 16, ff=128)]},
    # what keeps every fast path out, and values at the edges: a width that is no multiple of 8, 32 query heads on
    # one key/value head, a window of one key and one longer than any sequence here, a temperature that steps at
    # every position, one key channel group of 300 and value heads of 1 030 lanes, ranks and head counts of 1,
    # tau 1, an attention layer without a feed-forward, no soft cap
    "W": {"architecture": "Romepel", "vocab": 97, "width": 100, "max_positions": 900, "norm": {"eps": 1e-5},
          "layers": [att(32, 1, 8, 6, 0.5, window=1),
                     gla(1, 300, 10, 1.0, 1, ff=50),
                     att(3, 3, 10, 10, 0.3, window=5000, q_temp=(1.5, 1), ff=36),
                     gla(2, 8, 1030, 2.5, 3)]},
}


def write_folder(path, cfg_dict, seed, store, sharpen=3.0):
    """A model folder with random weights; the query and key matrices are scaled up so that attention is not
    close to uniform and a key that is wrongly seen or missed changes the logits."""
    config = config_from_dict(cfg_dict)
    tensors = random_tensors(parameter_list(config.model_spec()), seed, store)
    for name in list(tensors):
        if name.endswith((".mix.q", ".mix.k")):
            tensors[name] = (tensors[name].float() * sharpen).to(store)
        if name.endswith((".mix.v", ".mix.o", ".mlp.up", ".mlp.down", "embed", "pos", "head")):
            tensors[name] = (tensors[name].float() * 3.0).to(store)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config.to_dict()))
    write_safetensors(path / "model.safetensors", tensors, {"format": "pt"})
    return path


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("romepel")
    return {(name, dtype): write_folder(root / f"{name}_{dtype}", cfg, 7 + i, STORE[dtype])
            for i, (name, cfg) in enumerate(CONFIGS.items()) for dtype in DTYPES}


def toks(cfg, n, seed):
    return np.random.RandomState(seed).randint(0, cfg["vocab"], size=n).tolist()


# -- mechanisms alone -----------------------------------------------------------------------------

def test_norm_with_weights_around_zero_and_added_into_the_stream():
    g = torch.Generator().manual_seed(1)
    x, w, res = torch.randn(9, 88, generator=g) * 3, torch.randn(88, generator=g) * 0.1, torch.randn(9, 88, generator=g)
    want = P.offset_norm(x.double().numpy(), w.double().numpy(), 2e-6)
    out = torch.empty(9, 88, device=DEV)
    ops.rmsnorm(x.to(DEV), w.to(DEV), 2e-6, out, gamma_offset=1.0)
    check(out, want, 1e-6, "norm with offset")
    stream = res.to(DEV)
    ops.rmsnorm(x.to(DEV), w.bfloat16().to(DEV), 2e-6, stream, gamma_offset=1.0, accumulate=True)
    want = res.double().numpy() + P.offset_norm(x.double().numpy(), w.bfloat16().double().numpy(), 2e-6)
    check(stream, want, 1e-6, "norm added into the stream")


@pytest.mark.parametrize("dim", [88, 344, 1024, 2052, 8192])
def test_closing_and_opening_norm_in_one_pass(dim):
    """r += norm(b) * (1 + w1); y = norm(r) * (1 + w2) against the two norms one after the other."""
    g = torch.Generator().manual_seed(dim)
    b, r = torch.randn(5, dim, generator=g) * 2, torch.randn(5, dim, generator=g)
    w1, w2 = torch.randn(dim, generator=g) * 0.1, torch.randn(dim, generator=g) * 0.1
    want_r = r.double().numpy() + P.offset_norm(b.double().numpy(), w1.double().numpy(), 1e-6)
    want_y = P.offset_norm(want_r, w2.double().numpy(), 3e-6)
    for out_dt in (torch.float32, torch.bfloat16):
        stream, y = r.to(DEV), torch.empty(5, dim, dtype=out_dt, device=DEV)
        ops.rmsnorm_pair(b.to(DEV), stream, w1.to(DEV), 1.0, 1e-6, w2.to(DEV), 1.0, 3e-6, y)
        check(stream, want_r, 1e-6, "the stream after the closing norm")
        check(y, want_y, 2e-6 if out_dt == torch.float32 else 1e-2, "the opening norm")


def test_xielu_both_branches_and_soft_cap():
    z = torch.linspace(-9, 9, 1001)
    for p, q in ((0.3, -0.7), (-2.0, 1.5)):
        params = torch.tensor([p, q])
        out = torch.empty(1001, device=DEV)
        ops.xielu(z.to(DEV), params.to(DEV), out)
        check(out, P.xielu(z.double().numpy(), p, q), 2e-6, "xielu")
        half = torch.empty(1001, dtype=torch.bfloat16, device=DEV)
        ops.xielu(z.to(DEV), params.bfloat16().to(DEV), half)
        pb, qb = params.bfloat16().double().tolist()
        check(half, P.xielu(z.double().numpy(), pb, qb), 5e-3, "xielu, bfloat16 out")
    x = (torch.randn(7, 33, generator=torch.Generator().manual_seed(2)) * 30).to(DEV)
    want = 11.0 * np.tanh(x.double().cpu().numpy() / 11.0)
    ops.softcap(x, 11.0)
    check(x, want, 1e-6, "soft cap")


@pytest.mark.parametrize("m", [1, 8, 16, 17, 40, 64, 100, 256, 300, 600, 1100])
def test_xielu_in_the_epilogue_of_the_tensor_core_products(m):
    """Every product kernel (few tokens, cluster, stream-K, persistent, pairs of SMs) with the activation on its
    accumulators, against the product in float32 followed by the activation's own kernel."""
    from nncpu_b200.parts import Runtime
    rt = Runtime(DEV, torch.bfloat16)
    g = torch.Generator().manual_seed(m)
    k, n = 192, 328
    x = (torch.randn(m, k, generator=g) * 2).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.2).bfloat16().to(DEV)
    bias = torch.randn(n, generator=g).bfloat16().to(DEV)
    params = torch.tensor([0.4, -0.3])
    a, b = torch.nn.functional.softplus(params).tolist()
    plain = torch.empty(m, n, device=DEV)
    rt.linear(x, w, bias, plain)
    want = torch.empty(m, n, device=DEV)
    ops.xielu(plain, params.to(DEV), want)
    for out_dt in (torch.bfloat16, torch.float32):
        got = torch.empty(m, n, dtype=out_dt, device=DEV)
        rt.linear(x, w, bias, got, activation=("xielu", a, 0.5 + b))
        torch.cuda.synchronize()
        rt.check_status()
        check(got, want, 1e-5 if out_dt == torch.float32 else 8e-3, f"{m} tokens")


def test_embedding_with_learned_positions():
    g = torch.Generator().manual_seed(3)
    table, pos = torch.randn(50, 24, generator=g), torch.randn(30, 24, generator=g)
    ids = torch.tensor([4, 49, -1, 0], dtype=torch.int32)
    at = torch.tensor([0, 29, 3, 7], dtype=torch.int32)
    out = torch.empty(4, 24, device=DEV)
    ops.embed(table.bfloat16().to(DEV), ids.to(DEV), out, 1.0, pos.bfloat16().to(DEV), at.to(DEV))
    want = table.bfloat16().float()[ids.clamp(min=0).long()] + pos.bfloat16().float()[at.long()]
    want[2] = 0
    check(out, want, 1e-6, "embedding plus position")


@pytest.fixture(params=[2, 4])
def scan_columns(request):
    """Both arrangements of the scan kernel, whatever the grid's size would choose."""
    ops.gla_scan_force_columns(request.param)
    yield request.param
    ops.gla_scan_force_columns(0)


@pytest.mark.parametrize("H,d,e", [(3, 20, 48), (1, 64, 128), (2, 130, 33), (4, 128, 64), (1, 300, 40)])
def test_gla_recurrence_alone_in_portions_and_batches(H, d, e, scan_columns):
    """Three sequences of unequal lengths in one step against each alone, then the same tokens cut into portions
    (2, 1, 5, ... tokens) with the state carried in the state area, against the plain recurrence."""
    g = torch.Generator().manual_seed(d)
    lens = [37, 5, 70]
    tau, n_slots = 5.0, 6
    data = []
    for T in lens:
        proj = torch.randn(T, 2 * H * (d + e), generator=g)
        z = torch.randn(T, H * d, generator=g) * 2 + 2
        q, k = (proj[:, i * H * d:(i + 1) * H * d].double().numpy().reshape(T, H, d) for i in (0, 1))
        v = proj[:, 2 * H * d:2 * H * d + H * e].double().numpy().reshape(T, H, e)
        alpha = P.sigmoid(z.double().numpy().reshape(T, H, d)) ** (1 / tau)
        want = P.gla_recurrence(q * d ** -0.5, k, v, alpha, np.zeros((H, d, e)))
        data.append((proj, z, want))
    state = torch.zeros(n_slots + 1, H, d, e, device=DEV)
    slots = [4, 0, 2]

    def run(pieces):          # pieces: list of (sequence index, first, last) run as one step
        proj = torch.cat([data[b][0][lo:hi] for b, lo, hi in pieces]).to(DEV)
        z = torch.cat([data[b][1][lo:hi] for b, lo, hi in pieces]).to(DEV)
        cu = torch.tensor(np.cumsum([0] + [hi - lo for _, lo, hi in pieces]), dtype=torch.int32, device=DEV)
        sl = torch.tensor([slots[b] for b, _, _ in pieces], dtype=torch.int32, device=DEV)
        o = torch.empty(proj.shape[0], H * e, device=DEV)
        ops.gla_scan(proj, z, state, sl, cu, o, len(pieces), H, d, e, d ** -0.5, tau)
        return o.cpu()

    whole = run([(b, 0, lens[b]) for b in range(3)])
    at = 0
    for b in range(3):
        check(whole[at:at + lens[b]].view(lens[b], H, e), data[b][2], 2e-5, f"sequence {b} in a batch")
        at += lens[b]
    state.zero_()
    done, outs = [0, 0, 0], [[], [], []]
    sizes = [2, 1, 5, 3, 2, 64, 2]
    i = 0
    while any(done[b] < lens[b] for b in range(3)):
        pieces = []
        for b in range(3):
            if done[b] < lens[b]:
                n = min(sizes[(i + b) % len(sizes)], lens[b] - done[b])
                pieces.append((b, done[b], done[b] + n))
        o = run(pieces)
        at = 0
        for b, lo, hi in pieces:
            outs[b].append(o[at:at + hi - lo])
            at += hi - lo
            done[b] = hi
        i += 1
    at = 0
    for b in range(3):
        assert torch.equal(torch.cat(outs[b]), whole[at:at + lens[b]]), "portions give other bits than the whole"
        at += lens[b]
    # the decode step's kernel (recurrence, norm and gate in one launch) against the scan followed by the output stage
    w = torch.randn(e, generator=g).to(DEV)
    for out_dt in (torch.float32, torch.bfloat16):
        state.zero_()
        state2 = torch.zeros_like(state)
        for t in range(5):
            proj = torch.cat([data[b][0][t:t + 1] for b in range(3)] + [data[0][0][:1]]).to(DEV)
            z = torch.cat([data[b][1][t:t + 1] for b in range(3)] + [data[0][1][:1]]).to(DEV)
            sl = torch.tensor(slots + [-1], dtype=torch.int32, device=DEV)
            got = torch.empty(4, H * e, dtype=out_dt, device=DEV)
            ops.gla_step(proj, z, state, sl, w, 1e-5, got, H, d, e, d ** -0.5, tau)
            o = torch.empty(4, H * e, device=DEV)
            ops.gla_scan(proj, z, state2, sl, torch.arange(5, dtype=torch.int32, device=DEV), o, 4, H, d, e, d ** -0.5, tau)
            want = torch.empty(4, H * e, dtype=out_dt, device=DEV)
            ops.gla_output(o, proj, w, 1e-5, want, H, d, e)
            check(got[:3], want[:3], 1e-5 if out_dt == torch.float32 else 1e-2, f"decode step {t}")
            assert float(got[3].float().abs().max()) == 0, "a padding row is not zero"
        check(state, state2, 1e-6, "the state after five decode steps")
    at = 0
    for b in range(3):
        at += lens[b]
    assert float(state[n_slots].abs().max()) == 0 and float(state[1].abs().max()) == 0, "a foreign state row was written"


def test_gla_remembers_a_token_far_back_and_padding_leaves_the_state_alone():
    """One strong key/value pair at position 3, 600 weak tokens, decays near one on its channel: the query at
    the end that asks for that key must get its value back; a padding sequence (slot -1) gets zeros."""
    H, d, e, T, tau = 2, 24, 80, 604, 12.0
    g = torch.Generator().manual_seed(5)
    proj = torch.randn(T, 2 * H * (d + e), generator=g) * 0.05
    z = torch.full((T, H * d), 9.0)
    proj[3, H * d + 7] = 30.0                   # head 0, key channel 7
    proj[3, 2 * H * d:2 * H * d + e] = torch.arange(e).float()
    proj[T - 1, 0:d] = 0
    proj[T - 1, 7] = 5.0
    q, k = (proj[:, i * H * d:(i + 1) * H * d].double().numpy().reshape(T, H, d) for i in (0, 1))
    v = proj[:, 2 * H * d:2 * H * d + H * e].double().numpy().reshape(T, H, e)
    alpha = P.sigmoid(z.double().numpy().reshape(T, H, d)) ** (1 / tau)
    want = P.gla_recurrence(q * d ** -0.5, k, v, alpha, np.zeros((H, d, e)))
    state = torch.zeros(3, H, d, e, device=DEV)
    o = torch.empty(T + 1, H * e, device=DEV)
    ext = torch.cat([proj, proj[:1]]).to(DEV)
    zz = torch.cat([z, z[:1]]).to(DEV)
    cu = torch.tensor([0, 500, 501], dtype=torch.int32, device=DEV)
    ops.gla_scan(ext[:501].contiguous(), zz[:501].contiguous(), state, torch.tensor([1, -1], dtype=torch.int32, device=DEV),
                 cu, o[:501], 2, H, d, e, d ** -0.5, tau)
    assert float(o[500].abs().max()) == 0 and float(state[2].abs().max()) == 0 and float(state[0].abs().max()) == 0
    for t in range(500, T):                     # the rest token by token, as decoding does
        ops.gla_scan(ext[t:t + 1].contiguous(), zz[t:t + 1].contiguous(), state, torch.tensor([1], dtype=torch.int32, device=DEV),
                     torch.tensor([0, 1], dtype=torch.int32, device=DEV), o[t:t + 1], 1, H, d, e, d ** -0.5, tau)
    got = o[:T].cpu().view(T, H, e)
    assert abs(want[T - 1, 0, e - 1]) > 10 * np.abs(want[T - 2, 0]).max(), "the test's far token does not stand out"
    check(got[T - 1], want[T - 1], 1e-4, "the far token's value")
    check(got, want, 1e-4, "all rows")


def test_gla_output_stage():
    H, d, e, T = 3, 20, 48, 11
    g = torch.Generator().manual_seed(6)
    o, proj, w = torch.randn(T, H * e, generator=g) * 4, torch.randn(T, 2 * H * (d + e), generator=g), torch.randn(e, generator=g)
    gate = proj[:, 2 * H * d + H * e:].double().numpy()
    want = (P.rms(o.double().numpy().reshape(T, H, e), 1e-5) * w.double().numpy()).reshape(T, H * e) * P.silu(gate)
    out = torch.empty(T, H * e, device=DEV)
    ops.gla_output(o.to(DEV), proj.to(DEV), w.to(DEV), 1e-5, out, H, d, e)
    check(out, want, 2e-6, "norm and gate of the heads")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,vd,window", [(6, 2, 24, 40, 17), (4, 4, 16, 12, 0), (5, 1, 32, 32, 70),
                                                 (4, 2, 64, 64, 100), (2, 1, 128, 128, 64), (8, 2, 64, 64, 48)])
def test_biased_attention_alone(dtype, nh, nkv, hd, vd, window):
    """Queries at the end of two sequences (a prompt's portion of 9 tokens, one decoded token) over shuffled pages:
    distance bias per head, value heads of their own size, a window or none."""
    dt = STORE[dtype]
    lens = [150, 67]
    g = torch.Generator().manual_seed(hd + vd)
    kp, _, table, ks, _ = scatter_pages(9, nkv, hd, lens, dt, seed=1)
    _, vp, _, _, vs = scatter_pages(9, nkv, vd, lens, dt, seed=1)      # same page order (same seed), other width
    new = [9, 1]
    q = [torch.randn(n, nh, hd, generator=g).to(dt) for n in new]
    tok_seq = torch.tensor([0] * 9 + [1], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(list(range(lens[0] - 9, lens[0])) + [lens[1] - 1], dtype=torch.int32, device=DEV)
    out = torch.empty(10, nh * vd, dtype=dt, device=DEV)
    ops.attention(torch.cat(q).view(10, -1).to(DEV), kp, vp, table, tok_seq, tok_pos, out, nh, nkv, hd, 0.2, window, vd, 8.0)
    want = torch.cat([torch.from_numpy(P.biased_attention(
        q[b].double().numpy(), ks[b].double().numpy(), vs[b].double().numpy(), range(lens[b] - new[b], lens[b]), 0.2,
        window or None, P.head_slopes(nh))) for b in range(2)]).view(10, -1)
    check(out, want, 2e-5 if dtype == "float32" else 2e-2, "attention with distance bias")


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 64, 100), (2, 1, 128, 64), (8, 2, 64, 56), (16, 1, 64, 0), (12, 4, 128, 200),
                                              (6, 2, 64, 30), (3, 1, 128, 0), (5, 5, 64, 70), (1, 1, 64, 3)])
def test_biased_attention_on_the_tensor_core_kernels(nh, nkv, hd, window):
    """The bfloat16 kernels for prompts and for decode steps with the distance bias: three sequences (a portion of
    9 tokens, a whole prompt of 67, a portion of 130 that crosses two pages), then one token each, with the keys in
    one split and in two."""
    lens, new = [150, 67, 300], [9, 67, 130]
    g = torch.Generator().manual_seed(nh + hd)
    kp, vp, table, ks, vs = scatter_pages(12, nkv, hd, lens, torch.bfloat16, seed=3)
    slopes = P.head_slopes(nh)
    q = [torch.randn(n, nh, hd, generator=g).bfloat16() for n in new]
    n = sum(new)
    cu = torch.tensor(np.cumsum([0] + new), dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([p for b in range(3) for p in range(lens[b] - new[b], lens[b])], dtype=torch.int32, device=DEV)
    out = torch.empty(n, nh * hd, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill_mma(torch.cat(q).view(n, -1).to(DEV), kp, vp, table, cu, tok_pos, out, 3, nh, nkv, hd, 0.2, window, 8.0)
    want = torch.cat([torch.from_numpy(P.biased_attention(
        q[b].double().numpy(), ks[b].double().numpy(), vs[b].double().numpy(), range(lens[b] - new[b], lens[b]), 0.2,
        window or None, slopes)) for b in range(3)]).view(n, -1)
    check(out, want, 2e-2, "prompt kernel with distance bias")
    if ops.attention_prefill_tc_supported(nh, nkv, hd):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out_tc = torch.empty_like(out)
        ops.attention_prefill_tc(torch.cat(q).view(n, -1).to(DEV), kp, vp, table, cu, tok_pos, out_tc, status, 3, nh, nkv, hd,
                                 0.2, window, 8.0)
        assert int(status.item()) == 0
        check(out_tc, want, 2e-2, "tcgen05 prompt kernel with distance bias")
    last = torch.stack([q[b][-1] for b in range(3)]).view(3, -1).to(DEV)
    seq = torch.arange(3, dtype=torch.int32, device=DEV)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    want = torch.stack([want[int(cu[b + 1]) - 1] for b in range(3)])
    for n_splits in (1, 2):
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(ops.attention_decode_scratch_floats(3, nh, nkv, hd, n_splits), device=DEV)
        got = torch.empty(3, nh * hd, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode_mma(last, kp, vp, table, seq, pos, got, scratch, nh, nkv, hd, 0.2, window, n_splits, 8.0)
        check(got, want, 2e-2, f"decode kernel with distance bias, {n_splits} splits")


@pytest.mark.parametrize("window", [1, 5, 64, 65, 100])
def test_window_edge_one_key_inside_one_outside(window):
    """One key's score stands out (its query and key are scaled up).  At distance window - 1 it is seen and the
    output is its value; at distance window it is not, and the output must not know it.  At the end of a prompt's
    portion and for a decoded token, with the key on the far side of a page border too."""
    nh, nkv, hd, vd, n = 2, 1, 16, 24, 300
    for query in (n - 1, 2 * PAGE, 2 * PAGE + window - 1):
        for inside in (True, False):
            far = query - (window - 1 if inside else window)
            if far < 0:
                continue
            kp, _, table, ks, _ = scatter_pages(6, nkv, hd, [n], torch.float32, seed=2)
            _, vp, _, _, vs = scatter_pages(6, nkv, vd, [n], torch.float32, seed=2)
            q = torch.randn(1, nh, hd, generator=torch.Generator().manual_seed(window)) * 0.1
            q[0, :, 3] = 40.0
            page, row = int(table[0, far // PAGE]), far % PAGE
            kp[page, 0, row] = 0
            kp[page, 0, row, 3] = 40.0
            ks[0][far] = kp[page, 0, row].cpu()
            out = torch.empty(1, nh * vd, device=DEV)
            args = (table, torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([query], dtype=torch.int32, device=DEV))
            ops.attention(q.view(1, -1).to(DEV), kp, vp, *args, out, nh, nkv, hd, 1.0, window, vd, 8.0)
            want = P.biased_attention(q.double().numpy(), ks[0][:query + 1].double().numpy(),
                                      vs[0][:query + 1].double().numpy(), [query], 1.0, window, P.head_slopes(nh))
            check(out.view(1, nh, vd), want, 1e-5, f"window {window}, query {query}, key {'inside' if inside else 'outside'}")
            hit = float((out.view(nh, vd)[0].cpu() - vs[0][far, 0]).abs().max())
            assert (hit < 1e-3) == inside, f"window {window}: the key at distance {query - far} is {'missed' if inside else 'seen'}"


def test_query_temperature_steps_where_it_should():
    """q at position p is multiplied by 1 + c ln(floor((p + 1) / every) + 1): positions every - 2, every - 1 (the
    first with a factor above one), 2 every - 1."""
    nh, hd, every, c = 2, 8, 6, 0.7
    pos = [0, every - 2, every - 1, 2 * every - 2, 2 * every - 1, 100]
    n = len(pos)
    qkv = torch.ones(n, nh * hd, device=DEV)
    q_out = torch.empty(n, nh * hd, device=DEV)
    z = torch.zeros(n, dtype=torch.int32, device=DEV)
    ops.qk_norm_rope_append(qkv, None, None, 0.0, None, z, torch.tensor(pos, dtype=torch.int32, device=DEV), None, None,
                            None, q_out, nh, 0, hd, 0, (c, every))
    want = P.query_temperature(pos, c, every)
    assert want[1] == 1.0 and want[2] > 1.3 and want[3] == want[2] and want[4] > want[3]
    check(q_out[:, 0], want, 1e-6, "query temperature")


# -- the model ------------------------------------------------------------------------------------

def close(got, want, dtype, what):
    """Logits against the plain model's.  float32: the largest difference within 1e-4 of the largest logit.
    bfloat16: rounding of the activations to 8 bits of mantissa is the design's own noise, so the measure is the
    root mean square of a row's differences (measured here: 1 to 2 % of the logits' own over many rows, up to 3 % in
    single rows; held to 4 %) and the largest one is held to 8 %; a fault of the cache or of a window moves far
    more than that with these weights, and the float32 runs hold the same code to 1e-4."""
    if dtype == "float32":
        return check(got, want, TOL[dtype], what)
    g = got.detach().double().cpu().numpy()
    w = np.asarray(want, dtype=np.float64).reshape(g.shape)
    assert np.isfinite(g).all(), f"{what}: NaN or infinity"
    rms = float(np.sqrt(np.mean((g - w) ** 2)) / np.sqrt(np.mean(w ** 2)))
    assert rms <= 4e-2, f"{what}: root mean square of the differences {rms:.3e} of the logits' own"
    check(got, want, 8e-2, what)


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
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_token_by_token_against_the_whole(folders, name, dtype):
    """The same 200 tokens: whole; in portions of 2, 3, 64, 1, 65, ... tokens; a prompt of 40 and then one token a
    step for 160 steps (across windows and page borders).  All against the plain model; in float32 the three
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
    s3 = engine.alloc_slot()                 # the slot, pages and state row that the whole run used
    engine.step([s3], [t[:40]], [[]])
    rows = [engine.step([s3], [[t[i]]]).clone() for i in range(40, 200)]
    decoded = torch.cat(rows)
    close(decoded, want[40:], dtype, "token by token")
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
    for b in range(4):
        close(out[b], want[b][lens[b] - 1], dtype, f"prompt {b}")
    live = list(range(4))
    newcomer = toks(cfg, 90, 99)
    want_new = plain_logits(folders[name, dtype], newcomer)
    for step in range(24):
        live = [b for b in live if step < tails[b]]
        out = engine.step([slots[b] for b in live], [[seqs[b][lens[b] + step]] for b in live])
        for i, b in enumerate(live):
            close(out[i], want[b][lens[b] + step], dtype, f"sequence {b}, decoded token {step}")
        for b in list(range(4)):
            if step + 1 == tails[b] and b in live and tails[b] < 24:
                engine.free_slot(slots[b])
        if step == 11:                      # both short sequences are gone: their slots, pages and state rows are used again
            s = engine.alloc_slot()
            got = engine.step([s], [newcomer], [[0, 1, 63, 64, 89]])
            close(got, want_new[[0, 1, 63, 64, 89]], dtype, "a newcomer on used slots")
            engine.free_slot(s)
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_the_end_of_the_position_table(folders, dtype):
    """500 decoded tokens after a prompt of 150 (windows, pages and the temperature's steps pass by), up to the
    last position the table of learned positions has; one more token is refused before anything changes."""
    cfg = CONFIGS["R"]
    n = cfg["max_positions"]
    t = toks(cfg, n, 5)
    want = plain_logits(folders["R", dtype], t)
    model = Model.load(folders["R", dtype], dtype=dtype)
    engine = Engine(model, max_tokens=1024)
    assert engine.max_seq_len == n
    s = engine.alloc_slot()
    engine.step([s], [t[:150]], [[]])
    for i in range(150, n):
        out = engine.step([s], [[t[i]]])
        if i % 7 == 0 or i > n - 20:
            close(out[0], want[i], dtype, f"decoded position {i}")
    from nncpu_b200.errors import ContextFull
    with pytest.raises(ContextFull):
        engine.step([s], [[1]])
    assert engine.cache.length(s) == n


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_session(folders, name):
    """``Session.generate`` (scheduler, batches, captured decode steps) against greedy decoding of the plain model."""
    cfg = CONFIGS[name]
    folder = folders[name, "float32"]
    pcfg, w = P.load(folder)
    prompts = [toks(cfg, 70, 21), toks(cfg, 3, 22), toks(cfg, 129, 23)]
    want = []
    for p in prompts:
        seq = P.Sequence()
        logits = P.forward(pcfg, w, p, seq)
        out = []
        for _ in range(12):
            out.append(int(np.argmax(logits[-1])))
            logits = P.forward(pcfg, w, [out[-1]], seq)
        want.append(out)
    model = Model.load(folder, dtype="float32")
    session = Session(model, SessionParams(n_ctx=256, seed=1, max_batch=2))
    res = session.generate(prompts, GenerateParams(12, SamplerParams.greedy()), stop_token_ids=())
    assert [r.tokens for r in res] == want
    # the same in bfloat16: the first token of every reply (later ones may part ways by rounding)
    model = Model.load(folders[name, "bfloat16"], dtype="bfloat16")
    session = Session(model, SessionParams(n_ctx=256, seed=1, max_batch=3))
    res = session.generate(prompts, GenerateParams(4, SamplerParams.greedy()), stop_token_ids=())
    assert all(len(r.tokens) == 4 for r in res)


def test_model_folder_as_other_tools_write_it(tmp_path):
    """A file that does not name the decay projection's rank: the tensors decide it."""
    cfg = json.loads(json.dumps(CONFIGS["R"]))
    folder = write_folder(tmp_path / "m", cfg, 3, torch.float32)
    d = json.loads((folder / "config.json").read_text())
    for layer in d["layers"]:
        layer["mixer"].pop("rank", None)
    (folder / "config.json").write_text(json.dumps(d))
    t = toks(cfg, 20, 1)
    model = Model.load(folder, dtype="float32")
    engine = Engine(model, max_tokens=64)
    got = engine.step([engine.alloc_slot()], [t], [list(range(20))])
    check(got, plain_logits(folder, t), TOL["float32"], "rank from the file")
    assert model.info()["architecture"] == "Romepel"


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
    cfg.write_text(json.dumps(CONFIGS["R"]))
    run(run_random_weights, ["--random-weights", str(cfg), "5", str(tmp_path / "m"), "--fp32"])
    info = json.loads(run(run_info, ["--info", str(tmp_path / "m")]))
    assert info["config"]["architecture"] == "Romepel" and info["parameters"] > 0
    prompt = toks(CONFIGS["R"], 40, 3)
    got = [int(t) for t in run(run_gen, ["--gen", str(tmp_path / "m"), " ".join(map(str, prompt)), "8", "--fp32"]).splitlines()[0].split()]
    pcfg, w = P.load(tmp_path / "m")
    seq = P.Sequence()
    logits = P.forward(pcfg, w, prompt, seq)
    want = []
    for _ in range(8):
        want.append(int(np.argmax(logits[-1])))
        logits = P.forward(pcfg, w, [want[-1]], seq)
    assert got == want
    out = run(run_generate, ["-m", str(tmp_path / "m"), "--tokens", " ".join(map(str, prompt)), "-n", "6", "--temp", "0.8",
                             "--top-k", "20", "-s", "4", "-b", "3"]).split()
    assert len(out) >= 6 and all(0 <= int(t) < CONFIGS["R"]["vocab"] for t in out[:6])
