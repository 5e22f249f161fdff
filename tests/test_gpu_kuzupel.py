"""Kuzupel on the GPU against the plain implementation (tests/plain_kuzupel.py): every mechanism alone, the
kernels on inputs that make a wrong key, a window or a kept first token one off, a lost history or a lost
previous token show, and one model with everything fed whole, token by token, in portions and in mixed
batches over pools and slots that are used again."""
from __future__ import annotations

import math

import pytest
import torch

import kuzupel_cases as cases
import plain_kuzupel as plain

pytestmark = pytest.mark.gpu

F32_TOL = 5e-5          # float32 engine against the float64 plain implementation
BF16_TOL = 0.06         # bfloat16 engine against the plain implementation on the same (rounded) weights


def load(cfg, tensors, dtype):
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights.loader import load_tensors
    model = build_model(cfg, dtype)
    load_tensors(model, tensors, "cuda")
    return model


def replay(model, max_tokens=512, requests=4, page_size=16):
    from snowllm_b200.engine.replay import Replay
    return Replay(model, None, max_tokens, requests, page_size=page_size)


def reference(cfg, tensors, tokens, layers_out=None, **kw):
    return cases.plain_logits(cfg, {k: v.double() for k, v in tensors.items()}, tokens, layers_out, **kw)


def tolerance(dtype):
    return F32_TOL if dtype == "float32" else BF16_TOL


def engine_picks(rp):
    return [t.cpu() for n, t in rp.runner.taps if n == "moe_route"]


def routed_layers(cfg):
    return [i for i, l in enumerate(cfg["layers"]) if l["mlp"] is not None and l["mlp"]["kind"] == "moe"]


# --- each mechanism alone -------------------------------------------------------------------------

ALONE = {
    "slope_moe": dict(layers=[cases.slope_layer()]),
    "slope_one_kv_head_no_ff": dict(layers=[cases.slope_layer(heads=6, kv_heads=1, dim=8, vdim=4, window=5, mlp=None)]),
    "slope_causal_dense": dict(layers=[cases.slope_layer(heads=2, kv_heads=2, window=None, mlp=cases.dense(24, 0.5))]),
    "slope_tensor_core_sizes": dict(layers=[cases.slope_layer(heads=4, kv_heads=2, dim=32, vdim=16, window=37)]),
    "conv_dense": dict(layers=[cases.conv_layer()]),
    "conv_no_conv_no_rotation_no_kept": dict(layers=[cases.conv_layer(conv=None, rot_dims=0, keep_first=None, mlp=None)]),
    "conv_two_taps_whole_head_turns": dict(layers=[cases.conv_layer(heads=2, kv_heads=2, dim=8, vdim=8, conv=2, rot_dims=8,
                                                                    base=1e6, keep_first=0)]),
    "conv_one_tap": dict(layers=[cases.conv_layer(conv=1, window=7, keep_first=2, mlp=None)]),
    "conv_kept_more_than_window": dict(layers=[cases.conv_layer(window=6, keep_first=30, conv=7)]),
    "conv_causal": dict(layers=[cases.conv_layer(window=None, keep_first=None, conv=4)]),
    "conv_tensor_core_sizes": dict(layers=[cases.conv_layer(heads=4, kv_heads=2, dim=32, vdim=32, window=24, keep_first=9,
                                                            rot_dims=16, conv=4)]),
    "all_experts_picked_one_expert": dict(layers=[cases.slope_layer(mlp=cases.moe(8, 4, 4, 3.0, (24, 3.0))),
                                                  cases.conv_layer(mlp=cases.moe(16, 1, 1, 1.0, None))]),
    "no_pair_table_no_cap_no_scale": dict(layers=[cases.conv_layer(), cases.slope_layer()], pair=None, cap=None, mult=None,
                                          scale=1.0),
    "pair_table_of_one_bucket": dict(layers=[cases.slope_layer(mlp=None)], pair=(1, 0, 3), mult=1.3, cap=2.0),
    "heads_of_64": dict(layers=cases.HEADS_OF_64["layers"], width=64),
    "heads_of_128_and_unequal": dict(layers=[cases.conv_layer(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, window=70,
                                                              keep_first=17, conv=4, rot_dims=64),
                                             cases.slope_layer(heads=4, kv_heads=2, dim=128, vdim=64, scale=0.09, window=45),
                                             cases.slope_layer(heads=34, kv_heads=2, dim=16, vdim=16, scale=0.3, window=29,
                                                               mlp=None)], width=48),
    # sizes that are multiples of nothing: the products leave the tensor cores
    "odd_sizes": dict(layers=[cases.conv_layer(heads=5, kv_heads=5, dim=6, vdim=10, window=7, keep_first=4, conv=3, rot_dims=6,
                                               mlp=cases.moe(20, 7, 3, 1.0, (12, 0.7))),
                              cases.slope_layer(heads=3, kv_heads=1, dim=10, vdim=6, window=9, mlp=cases.dense(22, 0.9))],
                      width=36, vocab=50),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALONE))
def test_each_mechanism_alone(name, dtype):
    kw = dict(ALONE[name])
    cfg = cases.config(kw.pop("layers"), **kw)
    tensors = cases.draw_weights(cfg, seed=len(name))
    tokens = cases.tokens_for(cfg, 70)
    model = load(cfg, tensors, dtype)
    rp = replay(model)
    rp.runner.taps = []
    got = cases.run_cuts(rp, "a", tokens, [len(tokens)])
    # the plain experts are put on the engine's picks: a near tie may fall either way, the rest must agree
    routed = routed_layers(cfg)
    force = dict(zip(routed, [t.long().sort(-1).values for t in engine_picks(rp)]))
    assert len(force) == len(routed)
    want_layers, free = [], {}
    want = reference(cfg, tensors, tokens, want_layers, picks=force)
    reference(cfg, tensors, tokens, picks_out=free)
    for i in routed:
        differ = (free[i] != force[i]).any(-1).float().mean()
        assert float(differ) <= (0.0 if dtype == "float32" else 0.1), (i, float(differ))
    layers = [t for n, t in rp.runner.taps if n == "layer_out"]
    assert len(layers) == len(want_layers)
    for x, w in zip(layers, want_layers):
        assert cases.relative_error(x.cpu(), w) < tolerance(dtype)
    assert cases.worst_row_error(got, want) < tolerance(dtype) * 2
    # token by token through the cache and the state gives the same
    rp.runner.taps = None
    again = cases.run_cuts(rp, "b", tokens, [1] * len(tokens))
    assert cases.worst_row_error(again, want) < tolerance(dtype) * 2


# --- the attention kernel on keys that stand out ---------------------------------------------------

def plain_attention(q, k, v, scale, window, keep=0, slopes=None, one_more=False, gate=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv], float64: out [T, H, dv] through the plain mask and softmax."""
    T, H = q.shape[:2]
    G = k.shape[1]
    mask = plain.window_mask(T, window, keep)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).double()
    out = []
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale
        if slopes is not None:
            s = s - slopes[h] * dist
        o = plain.masked_softmax(s, mask, one_more) @ v[:, g]
        out.append(o if gate is None else o * torch.sigmoid(gate[:, h:h + 1]))
    return torch.stack(out, 1)


def paged(k, v, P, dtype, gen, spare=3):
    """Keys and values in pages of P in a scrambled order: (key pool, value pool, block table [1, pages])."""
    T, G = k.shape[:2]
    pages = -(-T // P)
    order = torch.randperm(pages + spare, generator=gen)[:pages].int()
    kpool = torch.zeros(pages + spare, G, P, k.shape[2], dtype=dtype, device="cuda")
    vpool = torch.zeros(pages + spare, G, P, v.shape[2], dtype=dtype, device="cuda")
    for t in range(T):
        kpool[order[t // P], :, t % P] = k[t].to(dtype)
        vpool[order[t // P], :, t % P] = v[t].to(dtype)
    return kpool, vpool, order.view(1, -1).cuda().contiguous()


def run_kernel(q, pools, P, scale, window, keep, slopes, one_more, gate, mode):
    """mode: 'rows' every row alone, 'tiles' rows of the request side by side, 'chunks' rows alone with their
    keys cut into chunks (the kept first keys in chunks of their own) and merged."""
    from snowllm_b200.ops import kernels
    kpool, vpool, table = pools
    T, H, dk = q.shape
    G, dv = kpool.shape[1], vpool.shape[3]
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    kw = dict(window=window, keep=keep, slopes=None if slopes is None else slopes.float().cuda(),
              sink=torch.zeros(H, device="cuda") if one_more else None)
    if gate is not None:
        kw.update(gate=gate.to(q.dtype).cuda().contiguous(), gate_col=0)
    if mode == "tiles":
        n = kernels.split_attention_tile_rows(H, G, 1, dk, dv, q.dtype, False)
        tiles = torch.tensor([[s, min(n, T - s)] for s in range(0, T, n)], dtype=torch.int32, device="cuda")
        kw.update(tiles=tiles, tile_rows=n)
    else:
        kw.update(tile_rows=kernels.split_attention_tile_rows(H, G, 1, dk, dv, q.dtype, True))
    if mode == "chunks":
        chunk = kernels.split_attention_decode_chunk(H, G, 1, dk, dv, q.dtype)
        most = 0
        for pos in range(T):
            lo = max(0, pos - window + 1) if window else 0
            kept = -(-min(keep, lo) // chunk)
            most = max(most, kept + pos // chunk - lo // chunk + 1)
        kw.update(num_chunks=most, chunk=chunk)
    return kernels.split_attention(q.cuda(), kpool, vpool, table, P, positions, torch.zeros_like(positions), scale, **kw)


# (dk, dv): the second pair is one that the tensor-core kernels take in bfloat16; (window, kept first keys): kept
# keys within one tile, and kept keys that span more than a chunk beside a window shorter than a tile
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["rows", "tiles", "chunks"])
@pytest.mark.parametrize("dk,dv", [(12, 20), (48, 64)])
@pytest.mark.parametrize("window,keep", [(77, 5), (21, 150), (130, 0)])
def test_attention_kernel_sees_its_window_and_the_kept_first_keys(dtype, mode, dk, dv, window, keep):
    """One key per chosen row is made to stand out: the last key inside the window owns its row, the first one
    outside must not be seen; the last kept key owns a row far away, the first key that is not kept is not
    seen.  Pages in a scrambled order; window and kept count are no multiples of the tile, page or chunk."""
    g = torch.Generator().manual_seed(5)
    T, H, G, P = 300, 4, 2, 16
    q = torch.randn(T, H, dk, generator=g).to(dtype)
    k = (torch.randn(T, G, dk, generator=g) * 0.1).to(dtype)
    v = torch.randn(T, G, dv, generator=g).to(dtype)
    gate = torch.randn(T, H, generator=g) * 2
    inside, outside = 250, 240
    edge_in, edge_out = inside - window + 1, outside - window          # both beyond the kept keys
    assert edge_in > keep + 1 and edge_out > keep + 1 and edge_in != edge_out
    k[edge_in, 0] = (q[inside, 1].float() * 6).to(dtype)               # head 1 -> kv head 0
    k[edge_out, 1] = (q[outside, 2].float() * 6).to(dtype)             # head 2 -> kv head 1
    if keep:
        k[keep - 1, 1] = (q[299, 3].float() * 6).to(dtype)             # the last kept key, for the last row
        k[keep, 0] = (q[290, 0].float() * 6).to(dtype)                 # the first that is not kept
    slopes = torch.tensor([0.01, 0.0, 0.02, 0.003])
    pools = paged(k, v, P, dtype, g)
    got = run_kernel(q, pools, P, 0.25, window, keep, slopes, True, gate, mode).cpu().double()
    gate_r = gate.to(dtype).double()
    want = plain_attention(q.double(), k.double(), v.double(), 0.25, window, keep, slopes.double(), True, gate_r)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol
    s_in = torch.sigmoid(gate_r[inside, 1])
    assert float((got[inside, 1] - s_in * v[edge_in, 0].double()).abs().max()) < 0.05       # the key owns the row
    s_out = torch.sigmoid(gate_r[outside, 2])
    assert float((got[outside, 2] - s_out * v[edge_out, 1].double()).abs().max()) > 0.1 * float(s_out)
    if keep:
        s3 = torch.sigmoid(gate_r[299, 3])
        assert float((got[299, 3] - s3 * v[keep - 1, 1].double()).abs().max()) < 0.05
        s0 = torch.sigmoid(gate_r[290, 0])
        assert float((got[290, 0] - s0 * v[keep, 0].double()).abs().max()) > 0.1 * float(s0)
    # the first row sees one key beside the extra term: e^s / (1 + e^s) of its value
    s = float((k[0, 0].double() @ q[0, 0].double()) * 0.25)
    share = math.exp(s) / (1 + math.exp(s)) * torch.sigmoid(gate_r[0, 0])
    assert float((got[0, 0] - share * v[0, 0].double()).abs().max()) < tol


@pytest.mark.parametrize("P", [16, 64])
@pytest.mark.parametrize("window,keep", [(77, 5), (21, 150), (130, 0), (300, 290), (None, 0)])
@pytest.mark.parametrize("plain_softmax", [False, True])
def test_prompt_kernel_on_tensor_memory_sees_its_window_and_the_kept_first_keys(P, window, keep, plain_softmax):
    """The tcgen05 prompt kernel (heads of 64, bfloat16, tiles of 128 rows and 128 keys) over several tiles:
    the last key inside the window owns its row, the first one outside is not seen; the last kept key owns a
    row far away, the first key that is not kept is not seen.  A second request of 40 rows sits beside it."""
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(11)
    T, T2, H, G, d = 700, 40, 4, 2, 64
    dtype = torch.bfloat16
    q = torch.randn(T, H, d, generator=g).to(dtype)
    k = (torch.randn(T, G, d, generator=g) * 0.05).to(dtype)
    v = torch.randn(T, G, d, generator=g).to(dtype)
    gate = None if plain_softmax else torch.randn(T, H, generator=g) * 2
    slopes = None if plain_softmax else torch.tensor([0.01, 0.0, 0.02, 0.003])
    inside, outside = 650, 640
    if window:
        edge_in, edge_out = inside - window + 1, outside - window
        k[edge_in, 0] = (q[inside, 1].float() * 1.5).to(dtype)
        k[edge_out, 1] = (q[outside, 2].float() * 1.5).to(dtype)
    if keep:
        k[keep - 1, 1] = (q[699, 3].float() * 1.5).to(dtype)
        k[keep, 0] = (q[690, 0].float() * 1.5).to(dtype)
    kpool, vpool, table = paged(k, v, P, dtype, g)
    # the second request: the first T2 rows again, in pages of its own
    k2pool, v2pool, table2 = paged(k[:T2], v[:T2], P, dtype, g, spare=0)
    n1 = kpool.shape[0]
    kpool, vpool = torch.cat((kpool, k2pool)), torch.cat((vpool, v2pool))
    tables = torch.zeros(2, table.shape[1], dtype=torch.int32, device="cuda")
    tables[0], tables[1, :table2.shape[1]] = table[0], table2[0] + n1
    tiles = [[0, s, min(128, T - s), s] for s in range(0, T, 128)] + [[1, T, T2, 0]]
    tiles = torch.tensor(tiles, dtype=torch.int32, device="cuda")
    qq = torch.cat((q, q[:T2])).cuda()
    gg = None if gate is None else torch.cat((gate, gate[:T2])).to(dtype).cuda().contiguous()
    out = torch.empty(T + T2, H, d, dtype=dtype, device="cuda")
    kernels.attention_prefill_tc_split(qq, kpool, vpool, tables, P, tiles, 0.25, out, window=window, keep=keep,
                                       slopes=None if slopes is None else slopes.cuda(),
                                       sink=None if plain_softmax else torch.zeros(H, device="cuda"), gate=gg)
    assert kernels.attention_tc_status() == 0
    got = out.cpu().double()
    gate_r = None if gate is None else gate.to(dtype).double()
    want = plain_attention(q.double(), k.double(), v.double(), 0.25, window, keep,
                           None if slopes is None else slopes.double(), not plain_softmax, gate_r)
    assert float((got[:T] - want).abs().max()) < 3e-2
    assert float((got[T:] - want[:T2]).abs().max()) < 3e-2                   # the request beside it: the same rows
    share = (lambda row, head: 1.0) if gate is None else (lambda row, head: float(torch.sigmoid(gate_r[row, head])))
    if window:
        assert float((got[inside, 1] - share(inside, 1) * v[edge_in, 0].double()).abs().max()) < 0.05
        if edge_out >= keep:                                                 # not one of the kept keys
            assert float((got[outside, 2] - share(outside, 2) * v[edge_out, 1].double()).abs().max()) > 0.1 * share(outside, 2)
    if keep:
        assert float((got[699, 3] - share(699, 3) * v[keep - 1, 1].double()).abs().max()) < 0.05
        if keep < 690 - window + 1:
            assert float((got[690, 0] - share(690, 0) * v[keep, 0].double()).abs().max()) > 0.1 * share(690, 0)


@pytest.mark.parametrize("P", [16, 64])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("window,keep", [(77, 5), (21, 300), (130, 0), (600, 290), (None, 0)])
@pytest.mark.parametrize("plain_softmax", [False, True])
def test_decode_kernel_by_tma_sees_its_window_and_the_kept_first_keys(P, d, window, keep, plain_softmax):
    """Rows that stand alone (every position of a sequence as its own row) on the TMA decode kernel: chunks of
    256 keys, the kept first keys in chunks of their own, merged in order."""
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(13)
    T, H, G = 700, 4, 2
    dtype = torch.bfloat16
    q = torch.randn(T, H, d, generator=g).to(dtype)
    k = (torch.randn(T, G, d, generator=g) * 0.05).to(dtype)
    v = torch.randn(T, G, d, generator=g).to(dtype)
    gate = None if plain_softmax else torch.randn(T, H, generator=g) * 2
    slopes = None if plain_softmax else torch.tensor([0.01, 0.0, 0.02, 0.003])
    inside, outside = 650, 640
    boost = 96.0 / d
    if window:
        edge_in, edge_out = inside - window + 1, outside - window
        k[edge_in, 0] = (q[inside, 1].float() * boost).to(dtype)
        k[edge_out, 1] = (q[outside, 2].float() * boost).to(dtype)
    if keep:
        k[keep - 1, 1] = (q[699, 3].float() * boost).to(dtype)
        k[keep, 0] = (q[690, 0].float() * boost).to(dtype)
    kpool, vpool, table = paged(k, v, P, dtype, g)
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    most = 0
    for pos in range(T):
        lo = max(0, pos - window + 1) if window else 0
        most = max(most, -(-min(keep, lo) // 256) + pos // 256 - lo // 256 + 1)
    out = torch.empty(T, H, d, dtype=dtype, device="cuda")
    kernels.attention_decode_tma_split(q.cuda(), kpool, vpool, table, P, positions, torch.zeros_like(positions), 0.25,
                                       most, out, window=window, keep=keep,
                                       slopes=None if slopes is None else slopes.cuda(),
                                       sink=None if plain_softmax else torch.zeros(H, device="cuda"),
                                       gate=None if gate is None else gate.to(dtype).cuda().contiguous())
    assert kernels.attention_decode_status() == 0
    got = out.cpu().double()
    gate_r = None if gate is None else gate.to(dtype).double()
    want = plain_attention(q.double(), k.double(), v.double(), 0.25, window, keep,
                           None if slopes is None else slopes.double(), not plain_softmax, gate_r)
    assert float((got - want).abs().max()) < 3e-2
    share = (lambda row, head: 1.0) if gate is None else (lambda row, head: float(torch.sigmoid(gate_r[row, head])))
    if window:
        assert float((got[inside, 1] - share(inside, 1) * v[edge_in, 0].double()).abs().max()) < 0.05
        if edge_out >= keep:                                                 # not one of the kept keys
            assert float((got[outside, 2] - share(outside, 2) * v[edge_out, 1].double()).abs().max()) > 0.1 * share(outside, 2)
    if keep:
        assert float((got[699, 3] - share(699, 3) * v[keep - 1, 1].double()).abs().max()) < 0.05
        if keep < 690 - window + 1:
            assert float((got[690, 0] - share(690, 0) * v[keep, 0].double()).abs().max()) > 0.1 * share(690, 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["rows", "tiles", "chunks"])
def test_attention_kernel_slopes_without_extra_term_or_gate(dtype, mode):
    """The plain softmax with a distance penalty per head: a steep slope leaves a row its own key, a slope of
    zero leaves the scores as they are."""
    g = torch.Generator().manual_seed(6)
    T, H, G, P, dk, dv, window = 200, 4, 4, 8, 16, 16, 141
    q = torch.randn(T, H, dk, generator=g).to(dtype)
    k = torch.randn(T, G, dk, generator=g).to(dtype)
    v = torch.randn(T, G, dv, generator=g).to(dtype)
    slopes = torch.tensor([0.0, 0.1, 1.0, 60.0])
    pools = paged(k, v, P, dtype, g)
    got = run_kernel(q, pools, P, 0.2, window, 0, slopes, False, None, mode).cpu().double()
    want = plain_attention(q.double(), k.double(), v.double(), 0.2, window, 0, slopes.double())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol
    assert float((got[:, 3] - v[:, 3].double()).abs().max()) < tol            # every other key is 60 or more away
    free = plain_attention(q.double(), k.double(), v.double(), 0.2, window)
    assert float((got[:, 0] - free[:, 0]).abs().max()) < tol
    assert float((want[:, 1] - free[:, 1]).abs().max()) > 0.05


# (dk, dv, columns before q): sizes the scalar kernel takes, and rows of 16-byte vectors (the vector kernel; with
# 48 heads a thread holds several vectors and the sum over the projection crosses warps)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,lead", [(5, 2, 10, 6, 2), (5, 1, 16, 8, 8), (48, 12, 64, 32, 0)])
def test_prepare_normalises_over_the_whole_projection(dtype, H, G, dk, dv, lead):
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(9)
    M, P = 9, 4
    width = lead + H * dk + G * dk + G * dv + (3 if lead == 2 else 8)
    q_off, k_off, v_off = lead, lead + H * dk, lead + H * dk + G * dk
    proj = torch.randn(M, width, generator=g).to(dtype)
    proj[:, q_off:q_off + dk] *= 5                                         # one head far larger than the others
    wq, wk = (1 + 0.3 * torch.randn(H * dk, generator=g)).to(dtype), (1 + 0.3 * torch.randn(G * dk, generator=g)).to(dtype)
    positions = torch.arange(M, dtype=torch.int32)
    table = torch.tensor([[3, 1, 0]], dtype=torch.int32)
    kpool = torch.zeros(4, G, P, dk, dtype=dtype, device="cuda")
    vpool = torch.zeros(4, G, P, dv, dtype=dtype, device="cuda")
    q = kernels.split_prepare(proj.cuda(), q_off, k_off, v_off, wq.cuda(), wk.cuda(), 1e-3, None, 0, 1.0,
                              positions.cuda(), torch.zeros(M, dtype=torch.int32, device="cuda"), table.cuda(), P,
                              kpool, vpool, H, G, 1, dk, dv, whole_norm=True)
    tol = 1e-5 if dtype == torch.float32 else 0.03
    full = proj.double()
    want_q = (plain.rms(full[:, q_off:k_off], 1e-3) * wq.double()).view(M, H, dk)
    want_k = (plain.rms(full[:, k_off:v_off], 1e-3) * wk.double()).view(M, G, dk)
    assert float((q.cpu().double() - want_q).abs().max()) < tol * max(1.0, float(want_q.abs().max()) / 4)
    per_head = plain.rms(full[:, q_off:k_off].view(M, H, dk), 1e-3)
    assert float((per_head - want_q).abs().max()) > 0.3                    # a norm per head is another thing
    for m in range(M):
        page = int(table[0, m // P])
        assert float((kpool[page, :, m % P].cpu().double() - want_k[m]).abs().max()) < tol
        assert float((vpool[page, :, m % P].cpu().double() - full[m, v_off:v_off + G * dv].view(G, dv)).abs().max()) < tol


# --- the short convolution --------------------------------------------------------------------------

def run_conv(rows, C, w, cuts, slot, state):
    from snowllm_b200.ops import kernels
    out, at = [], 0
    for n in cuts:
        cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        seg = torch.zeros(n, dtype=torch.int32, device="cuda")
        out.append(kernels.causal_conv(rows[at:at + n].contiguous().cuda(), C, w, state, cu,
                                       torch.tensor([at], dtype=torch.int32, device="cuda"),
                                       torch.tensor([slot], dtype=torch.int32, device="cuda"), seg).cpu())
        at += n
    return torch.cat(out, 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,L,extra", [(24, 4, 5), (7, 2, 0), (130, 7, 3), (16, 1, 0), (64, 4, 8), (40, 3, 0), (8, 2, 0)])
def test_conv_kernel_carries_its_history_and_starts_fresh_in_a_used_slot(dtype, C, L, extra):
    """Fed whole, in portions down to one and two tokens (shorter than the taps), and token by token; the slot
    holds another request's history beforehand; columns beyond the convolved ones are left alone."""
    g = torch.Generator().manual_seed(C * L)
    T = 60
    rows = torch.randn(T, C + extra, generator=g).to(dtype)
    w = torch.randn(C, L, generator=g).to(dtype)
    want = plain.causal_taps(rows[:, :C].double(), w.double())
    tol = 1e-5 if dtype == torch.float32 else 0.03
    for cuts in ([T], cases.cuts_of(T, [2, 1, 9, 1, 1, 3]), [1] * T, [40] + [1] * 20):
        state = torch.randn(3, max(L - 1, 0), C, generator=g).to(dtype).cuda()
        before = state.clone()
        got = run_conv(rows, C, w.cuda(), cuts, 1, state)
        assert float((got.double() - want).abs().max()) < tol * float(want.abs().max()), cuts
        assert torch.equal(state[0], before[0]) and torch.equal(state[2], before[2])
        if L > 1:
            assert torch.equal(state[1].cpu(), rows[T - (L - 1):, :C])     # the last rows as they were stored


def test_conv_kernel_serves_unequal_segments_side_by_side():
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(3)
    C, L = 20, 4
    w = torch.randn(C, L, generator=g).cuda()
    lens, starts, slots = [9, 30, 1, 2], [14, 0, 45, 1], [2, 0, 3, 1]
    rows = [torch.randn(s + n, C, generator=g) for s, n in zip(starts, lens)]
    state = torch.randn(5, L - 1, C, generator=g).cuda()
    alone = []
    for r, s, n, slot in zip(rows, starts, lens, slots):
        st = torch.zeros(5, L - 1, C).cuda()
        alone.append(run_conv(r, C, w, [s, n] if s else [n], slot, st)[s:])
        if s:
            state[slot] = r[s - (L - 1):s].cuda() if s >= L - 1 else torch.cat((torch.zeros(L - 1 - s, C), r[:s])).cuda()
    flat = torch.cat([r[s:] for r, s in zip(rows, starts)], 0).cuda()
    cu = torch.tensor([0, 9, 39, 40, 42], dtype=torch.int32, device="cuda")
    seg = torch.repeat_interleave(torch.arange(4), torch.tensor(lens)).int().cuda()
    got = kernels.causal_conv(flat, C, w, state, cu, torch.tensor(starts, dtype=torch.int32, device="cuda"),
                              torch.tensor(slots, dtype=torch.int32, device="cuda"), seg)
    assert torch.allclose(got.cpu(), torch.cat(alone, 0), rtol=1e-6, atol=1e-6)
    for r, slot in zip(rows, slots):
        assert torch.equal(state[slot].cpu(), r[-(L - 1):])


# --- router, embedding, residual sum, cap -----------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,E,k", [(5, 8, 4), (40, 5, 1), (70, 6, 6), (300, 16, 3)])
def test_router_weights_are_the_softmax_over_the_picked_logits(dtype, M, E, k):
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(M + E)
    H = 64
    x = torch.randn(M, H, generator=g).to(dtype)
    w = (torch.randn(E, H, generator=g) * 0.5).to(dtype)
    b = torch.randn(E, generator=g) * 2                            # a bias that changes the choice
    z = x.double() @ w.double().T + b.double()
    ids, wts = kernels.moe_route(x.cuda(), w.cuda(), b.float().cuda(), k, False, 1.0, "softmax_picked")
    order = torch.argsort(-z, dim=-1, stable=True)[:, :k]
    margin = (torch.sort(z, -1, descending=True).values[:, k - 1] - torch.sort(z, -1, descending=True).values[:, min(k, E - 1)]).abs()
    clear = margin > (1e-4 if dtype == torch.float32 else 0.05) if k < E else torch.ones(M, dtype=torch.bool)
    assert clear.float().mean() > 0.8
    assert torch.equal(ids.cpu().long().sort(-1).values[clear], order.sort(-1).values[clear])
    want = torch.softmax(torch.gather(z, 1, ids.cpu().long()), -1)
    assert float((wts.cpu().double() - want).abs().max()) < (1e-5 if dtype == torch.float32 else 0.02)
    assert float((wts.sum(-1) - 1).abs().max()) < 1e-5
    unbiased = torch.argsort(-(z - b.double()), dim=-1, stable=True)[:, :k].sort(-1).values
    if k < E:
        assert not torch.equal(unbiased, order.sort(-1).values)    # without the bias the choice is another


def test_pair_embedding_reads_the_token_before_across_steps_and_slots():
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(2)
    V, H, buckets, a, b = 40, 24, 13, 29, 5
    table, pairs = torch.randn(V, H, generator=g).cuda(), torch.randn(buckets + 1, H, generator=g).cuda()
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (9, 1, 6)]
    last = torch.full((5,), 17, dtype=torch.int32, device="cuda")          # what earlier requests left
    slots = [3, 0, 1]

    def want(tokens):
        rows = plain.hashed_pair_rows(tokens, buckets, a, b)
        return table.cpu()[torch.tensor(tokens)] * 2.5 + pairs.cpu()[rows]

    def step(parts):
        """parts: [(sequence index, first, count)] as one batch."""
        ids = torch.tensor([t for s, f, n in parts for t in seqs[s][f:f + n]], dtype=torch.int32, device="cuda")
        lens = [n for _, _, n in parts]
        cu = torch.tensor([sum(lens[:i]) for i in range(len(lens) + 1)], dtype=torch.int32, device="cuda")
        seg = torch.repeat_interleave(torch.arange(len(parts)), torch.tensor(lens)).int().cuda()
        start = torch.tensor([f for _, f, _ in parts], dtype=torch.int32, device="cuda")
        sl = torch.tensor([slots[s] for s, _, _ in parts], dtype=torch.int32, device="cuda")
        return kernels.pair_embedding(ids, table, pairs, buckets, a, b, seg, cu, start, sl, last, scale=2.5).cpu()
    got = step([(0, 0, 4), (1, 0, 1), (2, 0, 2)])
    assert torch.allclose(got, torch.cat((want(seqs[0])[:4], want(seqs[1]), want(seqs[2])[:2])), atol=1e-6)
    assert torch.allclose(got[4], table.cpu()[seqs[1][0]] * 2.5 + pairs.cpu()[buckets], atol=1e-6)   # a first token: the last row
    got = step([(2, 2, 1), (0, 4, 1)])                                     # single tokens read the state
    assert torch.allclose(got, torch.stack((want(seqs[2])[2], want(seqs[0])[4])), atol=1e-6)
    got = step([(0, 5, 4), (2, 3, 3)])
    assert torch.allclose(got, torch.cat((want(seqs[0])[5:], want(seqs[2])[3:])), atol=1e-6)
    assert last.tolist() == [seqs[1][-1], seqs[2][-1], 17, seqs[0][-1], 17]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,H", [(7, 40), (200, 64)])
def test_norm_adds_scaled_gated_and_routed_parts(dtype, M, H):
    """residual += m * (sigmoid(gate) * a + sum_j w_j y_j), then the norm: one kernel, both of its forms."""
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(M)
    k, m = 3, 0.55
    res = torch.randn(M, H, generator=g)
    a, y = torch.randn(M, H, generator=g), torch.randn(M * k, H, generator=g)
    gate = torch.randn(M, 16, generator=g) * 2
    w = torch.rand(M, k, generator=g)
    pos = torch.randperm(M * k, generator=g).int()
    gamma = (1 + 0.2 * torch.randn(H, generator=g)).to(dtype)
    moe = kernels.ExpertSum(y.cuda(), pos.cuda(), w.cuda())
    delta = kernels.ScaledDelta(kernels.DeltaSum(a.cuda(), moe, a_gate=gate.cuda()), m)
    r = res.clone().cuda()
    x = kernels.add_rmsnorm(r, delta, gamma.cuda(), 1e-4, dtype)
    routed = (w.double()[:, :, None] * y.double()[pos.long()].view(M, k, H)).sum(1)
    new = res.double() + m * (torch.sigmoid(gate[:, :1].double()) * a.double() + routed)
    assert float((r.cpu().double() - new).abs().max()) < 1e-5
    want = plain.rms(new, 1e-4) * gamma.double()
    assert float((x.cpu().double() - want).abs().max()) < (1e-5 if dtype == torch.float32 else 0.03)
    assert float((delta.dense().cpu().double() - (new - res.double())).abs().max()) < 1e-5
    # a plain tensor times the constant, on chosen rows: the residual stays
    rows = torch.tensor([M - 1, 0, 3], dtype=torch.int32, device="cuda")
    r2 = res.clone().cuda()
    x2 = kernels.add_rmsnorm(r2, kernels.ScaledDelta(a.cuda(), m), gamma.cuda(), 1e-4, dtype, rows=rows)
    want2 = plain.rms(res.double() + m * a.double(), 1e-4)[rows.cpu().long()] * gamma.double()
    assert float((x2.cpu().double() - want2).abs().max()) < (1e-5 if dtype == torch.float32 else 0.03)
    assert torch.equal(r2.cpu(), res)


def test_logit_cap():
    from snowllm_b200.ops import kernels
    z = torch.linspace(-100, 100, 1001).view(7, 143).contiguous()
    got = kernels.softcap(z.clone().cuda(), 11.0).cpu()
    assert float((got.double() - plain.soft_cap(z.double(), 11.0)).abs().max()) < 1e-5
    assert float(got.abs().max()) <= 11.0


# --- one model with everything ----------------------------------------------------------------------

@pytest.fixture(scope="module", params=["mixed", "heads_of_64"])
def mixed(request):
    cfg = cases.MIXED if request.param == "mixed" else cases.HEADS_OF_64
    tensors = cases.draw_weights(cfg, seed=3)
    return cfg, tensors


def forced_reference(cfg, tensors, tokens, model):
    """Plain logits with the experts on the picks the engine made for the whole prompt."""
    rp = replay(model, max_tokens=1024)
    rp.runner.taps = []
    cases.run_cuts(rp, "picks", tokens, [len(tokens)])
    force = dict(zip(routed_layers(cfg), [t.long().sort(-1).values for t in engine_picks(rp)]))
    return reference(cfg, tensors, tokens, picks=force)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_token_by_token_and_portions_agree(mixed, dtype):
    cfg, tensors = mixed
    model = load(cfg, tensors, dtype)
    tokens = cases.tokens_for(cfg, 150, seed=1)
    want = forced_reference(cfg, tensors, tokens, model)
    tol = tolerance(dtype) * 2
    rp = replay(model)
    whole = cases.run_cuts(rp, "w", tokens, [len(tokens)])
    assert cases.worst_row_error(whole, want) < tol
    for cuts in ([1] * len(tokens), cases.cuts_of(len(tokens), [2]), cases.cuts_of(len(tokens), [3, 16, 2, 31, 1, 17]),
                 [100] + [1] * 50, [64, 64, 22]):
        got = cases.run_cuts(rp, "c", tokens, cuts)
        assert cases.worst_row_error(got, want) < tol, cuts
        if dtype == "float32":
            assert cases.worst_row_error(got, whole) < 2e-5, cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [8, 64])
def test_mixed_batches_over_pages_and_slots_that_are_used_again(mixed, dtype, page_size):
    """Requests of unequal lengths in waves over a pool that holds only the live ones and four slots; prompt
    portions sit beside single tokens; every request equals its run alone."""
    cfg, tensors = mixed
    model = load(cfg, tensors, dtype)
    lengths = [70, 3, 41, 1, 97, 26, 64, 2, 55]
    prompts = [cases.tokens_for(cfg, n, seed=10 + i) for i, n in enumerate(lengths)]
    alone = replay(model, page_size=page_size)
    want = [cases.run_cuts(alone, "x", p, [len(p)]) for p in prompts]
    rp = replay(model, max_tokens=4 * 128, requests=4, page_size=page_size)
    portions = [7, 2, 16, 1, 33]
    state = {}                                        # request index -> tokens fed
    got = {i: [] for i in range(len(prompts))}
    waiting = list(range(len(prompts)))
    turn = 0
    while waiting or state:
        while waiting and len(state) < 4:
            state[waiting.pop(0)] = 0
        entries, end = [], []
        for j, (i, fed) in enumerate(sorted(state.items())):
            left = len(prompts[i]) - fed
            # the last ten tokens of a request one by one; before that portions of changing size
            n = 1 if left <= 10 else min(portions[(turn + j) % len(portions)], left - 10)
            entries.append({"id": f"r{i}", "tokens": prompts[i][fed:fed + n], "want": list(range(n))})
            state[i] = fed + n
            if state[i] == len(prompts[i]):
                end.append(f"r{i}")
        out = rp.step(entries, end).double()
        at = 0
        for e in entries:
            got[int(e["id"][1:])].append(out[at:at + len(e["tokens"])])
            at += len(e["tokens"])
        for name in end:
            del state[int(name[1:])]
        turn += 1
    for i in range(len(prompts)):
        assert cases.worst_row_error(torch.cat(got[i]), want[i]) < (2e-5 if dtype == "float32" else tolerance(dtype) * 2), i
    assert all(p.held() == 0 for p in rp.cache.groups.values()) and rp.cache.slots.free_count == 4


def test_long_decoding_past_every_window_and_page(mixed):
    cfg, tensors = mixed
    model = load(cfg, tensors, "float32")
    tokens = cases.tokens_for(cfg, 400, seed=7)
    want = forced_reference(cfg, tensors, tokens, model)
    rp = replay(model, max_tokens=448, requests=1)
    got = cases.run_cuts(rp, "d", tokens, [5] + [1] * 395, end=False)
    assert cases.worst_row_error(got, want) < F32_TOL * 2
    # a window group gave back what it passed, but for the pages of its kept first tokens (pages of 16)
    tables = rp.live["d"].tables
    for key, table in tables.items():
        window, kept = key[1] if isinstance(key[1], tuple) else (key[1], 0)
        first = (400 - window + 1) // 16
        assert all(p >= 0 for p in table[:-(-kept // 16)]) and all(p >= 0 for p in table[first:])
        assert all(p < 0 for p in table[-(-kept // 16):first])
    assert ("paged", (33, 20)) in tables or ("paged", (150, 140)) in tables
    rp.step([], ["d"])
    assert all(pool.held() == 0 for pool in rp.cache.groups.values())


def test_greedy_generation_through_the_engine(mixed, tmp_path):
    """The framework's own entry point: a model folder, the scheduler with portions of 16 tokens, captured
    decode steps; the tokens are the plain implementation's greedy ones."""
    import snowllm_b200
    from snowllm_b200.engine import Engine, SamplingParams
    cfg, tensors = mixed
    cases.write_folder(tmp_path, cfg, tensors)
    for eager in (True, False):
        engine = Engine(snowllm_b200.load(tmp_path, "float32", "cuda"), max_num_seqs=3, max_model_len=256,
                        prefill_chunk=16, enforce_eager=eager, page_size=16)
        prompts = [cases.tokens_for(cfg, n, seed=20 + n) for n in (37, 5, 60)]
        outs = engine.generate(prompts, SamplingParams(temperature=0, max_new_tokens=24))
        for p, o in zip(prompts, outs):
            assert len(o) == 24
            logits = reference(cfg, tensors, p + o)
            for i, tok in enumerate(o):
                row = logits[len(p) - 1 + i]
                assert float(row.max() - row[tok]) < 1e-3, (eager, i)
