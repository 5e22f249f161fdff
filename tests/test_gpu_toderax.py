"""Toderax on the GPU against the plain implementation (tests/plain_toderax.py): every mechanism alone, the
kernels on inputs that make a wrong key, a block edge one token off, a lost state or a lost sink show, and
one model with everything fed whole, token by token, in portions and in mixed batches over pools and slots
that are used again."""
from __future__ import annotations

import math

import pytest
import torch

import plain_toderax as plain
import toderax_cases as cases

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


# --- each mechanism alone -------------------------------------------------------------------------

ALONE = {
    "memory_moe": dict(layers=[cases.memory_layer()]),
    "memory_one_head_no_ff": dict(layers=[cases.memory_layer(heads=1, dim=4, vdim=40, mlp=None)]),
    "memory_wide_rows": dict(layers=[cases.memory_layer(heads=2, dim=40, vdim=8, mlp=cases.moe(8, 2, 2, 0.5, None))]),
    "pair_moe": dict(layers=[cases.pair_layer()]),
    "pair_causal_no_rotation": dict(layers=[cases.pair_layer(chunk=None, rot_dims=0, mlp=None)]),
    "pair_whole_head_turns": dict(layers=[cases.pair_layer(heads=6, kv_heads=1, dim=8, vdim=4, chunk=5, r_heads=1,
                                                           r_dim=8, r_vdim=8, decay=(0.999,), rot_dims=8, base=1e6)]),
    "pair_all_experts_picked": dict(layers=[cases.pair_layer(heads=2, kv_heads=2, chunk=64,
                                                             mlp=cases.moe(8, 4, 4, 3.0, (24, 3.0)))]),
    "one_stream_with_weights": dict(layers=[cases.pair_layer(), cases.memory_layer()], streams=1),
    "no_streams_one_group_no_scale": dict(layers=[cases.memory_layer(), cases.pair_layer(chunk=16)], streams=None,
                                          groups=1, scale=1.0),
    "eight_streams": dict(layers=[cases.pair_layer(mlp=None), cases.memory_layer()], streams=8, groups=2),
    # sizes that are multiples of nothing: the products leave the tensor cores
    "odd_sizes": dict(layers=[cases.pair_layer(heads=5, kv_heads=5, dim=6, vdim=10, chunk=7, r_heads=3, r_dim=10, r_vdim=6,
                                               decay=(0.5, 0.9, 0.99), rot_dims=6, mlp=cases.moe(20, 7, 3, 1.0, (12, 0.7))),
                              cases.memory_layer(heads=5, dim=6, vdim=14, mlp=cases.moe(12, 3, 2, 0.9, (20, 2.0)))],
                      width=36, vocab=50, groups=3, streams=2),
}


def engine_picks(rp):
    return [t.cpu() for n, t in rp.runner.taps if n == "moe_route"]


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
    routed = [i for i, l in enumerate(cfg["layers"]) if l["mlp"] is not None]
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

def plain_attention(q, k, v, scale, block, head_scale=None, sink=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv], float64: out [T, H, dv] through the plain mask and softmax."""
    T, H = q.shape[:2]
    G = k.shape[1]
    mask = plain.same_chunk_causal(T, block)
    out = []
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale * (1.0 if head_scale is None else head_scale[h])
        sk = torch.tensor(-math.inf, dtype=torch.float64) if sink is None else sink[h]
        out.append(plain.softmax_with_sink(s, mask, sk) @ v[:, g])
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


def run_kernel(q, pools, P, scale, block, head_scale, sink, mode):
    """mode: 'rows' every row alone, 'tiles' rows of the request side by side, 'chunks' rows alone with their
    keys cut into chunks and merged."""
    from snowllm_b200.ops import kernels
    kpool, vpool, table = pools
    T, H, dk = q.shape
    G, dv = kpool.shape[1], vpool.shape[3]
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    kw = dict(block=block, head_scale=None if head_scale is None else head_scale.float().cuda(),
              sink=None if sink is None else sink.float().cuda(), out_dtype=torch.float32)
    if mode == "tiles":
        n = kernels.split_attention_tile_rows(H, G, 1, dk, dv, q.dtype, False)
        tiles = torch.tensor([[s, min(n, T - s)] for s in range(0, T, n)], dtype=torch.int32, device="cuda")
        kw.update(tiles=tiles, tile_rows=n)
    else:
        kw.update(tile_rows=kernels.split_attention_tile_rows(H, G, 1, dk, dv, q.dtype, True))
    if mode == "chunks":
        chunk = kernels.split_attention_decode_chunk(H, G, 1, dk, dv, q.dtype)
        pos = torch.arange(T)
        lo = pos - pos % block if block else torch.zeros_like(pos)
        kw.update(num_chunks=int((pos // chunk - lo // chunk).max()) + 1, chunk=chunk)
    return kernels.split_attention(q.cuda(), kpool, vpool, table, P, positions, torch.zeros_like(positions), scale, **kw)


# (dk, dv): the second pair is one that the tensor-core kernels take in bfloat16
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["rows", "tiles", "chunks"])
@pytest.mark.parametrize("dk,dv", [(12, 20), (48, 64)])
def test_attention_kernel_sees_exactly_its_block(dtype, mode, dk, dv):
    """One key per row is made to stand out: on the first position of the row's block it owns the output, on
    the last position of the block before it must not be seen at all.  Pages in a scrambled order; the block
    is no multiple of the key tile, the page or the chunk, and one block spans a chunk's edge."""
    g = torch.Generator().manual_seed(5)
    T, H, G, P, block = 300, 4, 2, 16, 137
    q = torch.randn(T, H, dk, generator=g).to(dtype)
    k = (torch.randn(T, G, dk, generator=g) * 0.1).to(dtype)
    v = torch.randn(T, G, dv, generator=g).to(dtype)
    inside, outside, late = 250, 200, 299                      # rows of the block 137..273 and of 274..
    k[137, 0] = (q[inside, 1].float() * 6).to(dtype)            # the farthest key row 250 sees (head 1 -> kv head 0)
    k[136, 1] = (q[outside, 2].float() * 6).to(dtype)           # one before row 200's block (head 2 -> kv head 1)
    k[274, 1] = (q[late, 3].float() * 6).to(dtype)              # the first key of the last block
    head_scale = torch.tensor([1.0, 1.5, 2.0, 0.7])
    pools = paged(k, v, P, dtype, g)
    got = run_kernel(q, pools, P, 0.25, block, head_scale, None, mode).cpu().double()
    want = plain_attention(q.double(), k.double(), v.double(), 0.25, block, head_scale.double())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol
    assert float((want[inside, 1] - v[137, 0].double()).abs().max()) < 0.05      # the key owns the row
    assert float((got[inside, 1] - v[137, 0].double()).abs().max()) < 0.05
    assert float((got[late, 3] - v[274, 1].double()).abs().max()) < 0.05
    assert float((got[outside, 2] - v[136, 1].double()).abs().max()) > 0.3
    # the first rows of a sequence and of a block see one key: its value as it is
    for row, head in ((0, 0), (137, 2), (274, 1)):
        assert float((got[row, head] - v[row, head // 2].double()).abs().max()) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["rows", "tiles", "chunks"])
@pytest.mark.parametrize("dk,dv,block", [(20, 12, None), (32, 48, 290)])
def test_attention_kernel_finds_a_far_key_and_counts_the_sink_once(dtype, mode, dk, dv, block):
    """Rows over 300 keys in pages of 8.  Head 0 of the last row looks for the key at position 12 among
    hundreds; head 1's sink is so large that its output all but vanishes; head 2's so small that it does
    nothing; head 3 sits between (its share of the denominator is checked by the numbers).  The factor per
    head multiplies the scores but not the sink."""
    g = torch.Generator().manual_seed(8)
    T, H, G, P = 300, 4, 1, 8
    first = 0 if block is None else 290
    far = first + 3
    q = torch.randn(T, H, dk, generator=g).to(dtype)
    k = (torch.randn(T, G, dk, generator=g) * 0.2).to(dtype)
    v = (torch.randn(T, G, dv, generator=g) * 0.5).to(dtype)
    if block is None:
        far = 12
    looks = q[T - 1, 0].float()
    k[far, 0] = (looks * (100 / float(looks @ looks))).to(dtype)           # a score of 30 after the scale
    v[far, 0] = 1.5
    sink = torch.tensor([-30.0, 200.0, -200.0, 0.5])
    head_scale = torch.tensor([1.0, 1.0, 1.0, 3.0])
    pools = paged(k, v, P, dtype, g)
    got = run_kernel(q, pools, P, 0.3, block, head_scale, sink, mode).cpu().double()
    want = plain_attention(q.double(), k.double(), v.double(), 0.3, block, head_scale.double(), sink.double())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol
    if block is None:
        assert float((got[T - 1, 0] - 1.5).abs().max()) < 0.05            # the far key owns the row
    assert float(got[:, 1].abs().max()) < 1e-6                            # the sink took everything
    free = plain_attention(q.double(), k.double(), v.double(), 0.3, block, head_scale.double())
    assert float((got[:, 2] - free[:, 2]).abs().max()) < tol              # a sink far below does nothing
    assert float((want[:, 3] - free[:, 3]).abs().max()) > 0.01            # one in between takes its share
    # the first token of a sequence or block: one key, weight e^s / (e^s + e^sink), s with the head's factor
    s = float((k[first, 0].double() @ q[first, 3].double()) * 0.3 * 3.0)
    share = math.exp(s) / (math.exp(s) + math.exp(0.5))
    assert float((got[first, 3] - share * v[first, 0].double()).abs().max()) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prepare_adds_the_bias_normalises_without_a_weight_and_writes_the_rows(dtype):
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(9)
    M, H, G, dk, dv, P = 13, 4, 2, 10, 6, 4
    width = 3 + H * dk + G * dk + G * dv + 5
    q_off, k_off, v_off = 3, 3 + H * dk, 3 + H * dk + G * dk
    proj = torch.randn(M, width, generator=g).to(dtype)
    bias = torch.randn(width, generator=g)
    positions = torch.tensor([40, 41, 42, 0, 1, 2, 3, 4, 5, 6, 7, 8, 1000], dtype=torch.int32)
    row_seg = torch.tensor([0] * 3 + [1] * 9 + [2], dtype=torch.int32)
    table = torch.full((3, 251), 0, dtype=torch.int32)
    table[0, 10], table[1, 0], table[1, 1], table[1, 2], table[2, 250] = 5, 2, 7, 1, 3
    kpool = torch.zeros(8, G, P, dk, dtype=dtype, device="cuda")
    vpool = torch.zeros(8, G, P, dv, dtype=dtype, device="cuda")
    q = kernels.split_prepare(proj.cuda(), q_off, k_off, v_off, None, None, 1e-3, None, 0, 1.0, positions.cuda(),
                              row_seg.cuda(), table.cuda(), P, kpool, vpool, H, G, 1, dk, dv, proj_bias=bias.cuda(),
                              plain_norm=True)
    tol = 1e-5 if dtype == torch.float32 else 0.03
    full = proj.double() + bias.double()
    want_q = plain.rms(full[:, q_off:k_off].view(M, H, dk), 1e-3)
    want_k = plain.rms(full[:, k_off:v_off].view(M, G, dk), 1e-3)
    want_v = full[:, v_off:v_off + G * dv].view(M, G, dv)
    assert float((q.cpu().double() - want_q).abs().max()) < tol
    for m in range(M):
        pos = int(positions[m])
        page = int(table[int(row_seg[m]), pos // P])
        assert float((kpool[page, :, pos % P].cpu().double() - want_k[m]).abs().max()) < tol
        assert float((vpool[page, :, pos % P].cpu().double() - want_v[m]).abs().max()) < tol
    assert int((kpool.float().abs().sum(-1) > 0).sum()) == M * G                # nothing else was written


# --- the matrix memory ----------------------------------------------------------------------------

def pieces_of(lens, rows):
    """The segments of a step cut into pieces of up to ``rows`` rows, as the memory kernel takes them."""
    table, first_piece, first = [], [0], 0
    for b, n in enumerate(lens):
        cuts = list(range(0, n, rows))
        table += [(b, first + r, min(rows, n - r), int(r == 0) + 2 * int(r == cuts[-1])) for r in cuts]
        first_piece.append(len(table))
        first += n
    return (torch.tensor(table, dtype=torch.int32, device="cuda"),
            torch.tensor(first_piece, dtype=torch.int32, device="cuda"))


def run_memory(proj, cols, cuts, slot, state, H, dk, dv, piece_rows=None, **kw):
    """One request's rows through the memory kernel in steps of the sizes ``cuts`` (every step continues from
    the state slot; with ``piece_rows`` every step is cut into pieces that blocks of their own walk); the raw
    head outputs [T, H*dv]."""
    from snowllm_b200.ops import kernels
    out, at = [], 0
    for n in cuts:
        cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        start = torch.tensor([at], dtype=torch.int32, device="cuda")
        sl = torch.tensor([slot], dtype=torch.int32, device="cuda")
        extra = dict(kw)
        if piece_rows:
            extra["pieces"] = pieces_of([n], piece_rows)
        if "inv_freq" in kw:
            extra["positions"] = torch.arange(at, at + n, dtype=torch.int32, device="cuda")
        out.append(kernels.decay_memory(proj[at:at + n].contiguous().cuda(), *cols, cu, start, sl, state, H, dk, dv,
                                        **extra).cpu())
        at += n
    return torch.cat(out, 0)


@pytest.mark.parametrize("H,dk,dv", [(2, 12, 8), (3, 40, 40), (1, 32, 72), (2, 100, 20)])
def test_retention_kernel_carries_its_state_and_starts_fresh_in_a_used_slot(H, dk, dv):
    """Fixed decays (one of them 1: nothing is ever forgotten), part of each head turning.  Fed whole, in
    portions down to two tokens and token by token; the slot holds another request's state beforehand."""
    g = torch.Generator().manual_seed(H * dk)
    T, rot, base = 150, 8, 300.0
    width = 5 + 2 * H * dk + H * dv
    proj = torch.randn(T, width, generator=g)
    proj[3, 5 + H * dk:5 + 2 * H * dk] *= 8                             # a key far back that stands out
    decay = torch.tensor([1.0, 0.5, 0.98][:H])
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32).cuda()
    q = proj[:, 5:5 + H * dk].double().view(T, H, dk)
    k = proj[:, 5 + H * dk:5 + 2 * H * dk].double().view(T, H, dk)
    v = proj[:, 5 + 2 * H * dk:].double().view(T, H, dv)
    pos = torch.arange(T)
    qr, kr = plain.rotate_halves(q, pos, base, rot), plain.rotate_halves(k, pos, base, rot) * dk ** -0.5
    want = torch.cat([plain.decayed_memory(qr[:, h], kr[:, h], v[:, h], torch.full((T, dk), float(decay[h]),
                                                                                   dtype=torch.float64))
                      for h in range(H)], -1)
    cols = (5, 5 + H * dk, 5 + 2 * H * dk)
    kw = dict(decay=decay.cuda(), inv_freq=inv_freq, rot_dim=rot, k_scale=dk ** -0.5)
    scale = float(want.abs().max())
    for cuts in ([T], cases.cuts_of(T, [2, 31, 1, 33, 64]), [100] + [1] * 50):
        state = torch.randn(3, H, dk, dv, generator=g).cuda()          # what an earlier request left
        before = state.clone()
        got = run_memory(proj, cols, cuts, 1, state, H, dk, dv, **kw)
        assert float((got.double() - want).abs().max()) < 2e-5 * scale, cuts
        assert torch.equal(state[0], before[0]) and torch.equal(state[2], before[2])   # the other slots stay
        # the same steps in pieces (of one token, of a few, of exactly a step, of more than a step)
        for rows in (1, 7, 32, 64, 200):
            again = before.clone()
            got = run_memory(proj, cols, cuts, 1, again, H, dk, dv, piece_rows=rows, **kw)
            assert float((got.double() - want).abs().max()) < 2e-5 * scale, (cuts, rows)
            assert torch.equal(again[0], before[0]) and torch.equal(again[2], before[2])
            assert float((again[1] - state[1]).abs().max()) < 2e-5 * float(state[1].abs().max()), (cuts, rows)
    # the last state is the sum it should be: S = sum_j decay^(T-1-j) k_j v_j^T
    S = sum(float(decay[0]) ** (T - 1 - j) * torch.outer(kr[j, 0], v[j, 0]) for j in range(T))
    assert float((state[1, 0].cpu().double() - S).abs().max()) < 2e-5 * float(S.abs().max())


@pytest.mark.parametrize("H,dk,dv", [(2, 8, 12), (3, 36, 33), (1, 64, 64)])
def test_gated_memory_kernel_writes_what_it_forgets(H, dk, dv):
    g = torch.Generator().manual_seed(dk)
    T = 90
    width = 2 * H * dk + H * dv + 3
    proj = torch.randn(T, width, generator=g) * 1.5
    bias, low = torch.randn(H * dk, generator=g), torch.rand(H * dk, generator=g) * 0.95
    low[0], low[1] = 0.0, 0.999                                          # no bound, and all but a bound of one
    q = plain.silu(proj[:, :H * dk].double()).view(T, H, dk)
    f = (low.double() + (1 - low.double()) * torch.sigmoid(proj[:, H * dk:2 * H * dk].double() + bias.double())).view(T, H, dk)
    v = proj[:, 2 * H * dk:2 * H * dk + H * dv].double().view(T, H, dv)
    want = torch.cat([plain.decayed_memory(q[:, h], 1 - f[:, h], v[:, h], f[:, h]) for h in range(H)], -1)
    cols = (0, H * dk, 2 * H * dk)
    for cuts in ([T], cases.cuts_of(T, [2, 32, 1, 3]), [1] * T):
        state = torch.randn(2, H, dk, dv, generator=g).cuda()
        first = state.clone()
        got = run_memory(proj, cols, cuts, 0, state, H, dk, dv, gate_bias=bias.cuda(), gate_low=low.cuda())
        assert float((got.double() - want).abs().max()) < 2e-5 * float(want.abs().max()), cuts
        for rows in (1, 5, 33):
            again = first.clone()
            got = run_memory(proj, cols, cuts, 0, again, H, dk, dv, piece_rows=rows, gate_bias=bias.cuda(),
                             gate_low=low.cuda())
            assert float((got.double() - want).abs().max()) < 2e-5 * float(want.abs().max()), (cuts, rows)
            assert float((again[0] - state[0]).abs().max()) < 2e-5 * float(state[0].abs().max()), (cuts, rows)


def test_memory_kernel_serves_unequal_segments_side_by_side():
    """Three requests in one launch: a prompt's portion that continues, a fresh prompt in a slot that was used,
    and a single token; each equals its run alone."""
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(4)
    H, dk, dv = 2, 16, 24
    cols = (0, H * dk, 2 * H * dk)
    width = 2 * H * dk + H * dv
    decay = torch.tensor([0.9, 0.999]).cuda()
    lens, starts, slots = [37, 70, 1], [20, 0, 45], [2, 0, 3]
    rows = [torch.randn(s + n, width, generator=g) for s, n in zip(starts, lens)]
    state = torch.randn(4, H, dk, dv, generator=g).cuda()
    alone, kept = [], []
    for r, s, n, slot in zip(rows, starts, lens, slots):
        st = torch.zeros(4, H, dk, dv).cuda()
        alone.append(run_memory(r, cols, [s, n] if s else [n], slot, st, H, dk, dv, decay=decay)[s:])
        kept.append(st[slot].clone())
        if s:                                                            # the state its first portion left
            st2 = torch.zeros(4, H, dk, dv).cuda()
            run_memory(r[:s], cols, [s], slot, st2, H, dk, dv, decay=decay)
            state[slot] = st2[slot]
    flat = torch.cat([r[s:] for r, s in zip(rows, starts)], 0).cuda()
    cu = torch.tensor([0, 37, 107, 108], dtype=torch.int32, device="cuda")
    before = state.clone()
    got = kernels.decay_memory(flat, *cols, cu, torch.tensor(starts, dtype=torch.int32, device="cuda"),
                               torch.tensor(slots, dtype=torch.int32, device="cuda"), state, H, dk, dv, decay=decay)
    assert torch.allclose(got.cpu(), torch.cat(alone, 0), rtol=1e-5, atol=1e-5)
    for slot, st in zip(slots, kept):
        assert torch.allclose(state[slot], st, rtol=1e-5, atol=1e-5)
    # in pieces: segments of several pieces, of one piece and of one token side by side
    for rows in (8, 37, 64):
        again = before.clone()
        got = kernels.decay_memory(flat, *cols, cu, torch.tensor(starts, dtype=torch.int32, device="cuda"),
                                   torch.tensor(slots, dtype=torch.int32, device="cuda"), again, H, dk, dv,
                                   decay=decay, pieces=pieces_of(lens, rows))
        want = torch.cat(alone, 0)                                      # the same sums in another order
        assert float((got.cpu() - want).abs().max()) < 1e-5 * float(want.abs().max()), rows
        for slot, st in zip(slots, kept):
            assert float((again[slot] - st).abs().max()) < 1e-5 * float(st.abs().max()), rows
        assert torch.equal(again[1], before[1])


# --- streams, norms and the small kernels -----------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,W,groups", [(1, 40, 1), (3, 36, 3), (4, 100, 5), (8, 64, 64)])
def test_streams_norm_applies_the_pending_update_and_reads_the_streams(dtype, S, W, groups):
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(S + W)
    M, k, eps = 11, 2, 1e-3
    x0 = torch.randn(M, W, generator=g)
    w = (1 + 0.3 * torch.randn(W, generator=g)).to(dtype)
    sets = [{n: torch.randn(shape, generator=g).double() for n, shape in (("in", (S,)), ("out", (S,)), ("mix", (S, S)))}
            for _ in range(3)]
    tol = 1e-5 if dtype == torch.float32 else 0.04

    def f32(t):
        return t.float().cuda().contiguous()

    def normed(X, read):
        return plain.group_rms_norm(sum(read[s] * X[s] for s in range(S)), w.double(), groups, eps)

    # the first norm of a model: every stream starts as a copy of the embedding output
    streams = torch.empty(M, S, W, device="cuda")
    got = kernels.streams_norm(streams, w.cuda(), groups, eps, dtype, init=x0.cuda(), read=f32(sets[0]["in"]))
    X = [x0.double() for _ in range(S)]
    assert float((got.cpu().double() - normed(X, sets[0]["in"])).abs().max()) < tol
    assert all(torch.equal(streams[:, s].cpu(), x0) for s in range(S))
    # a plain output pending
    y = torch.randn(M, W, generator=g)
    pending = kernels.StreamsDelta(streams, y.cuda(), f32(sets[0]["mix"]), f32(sets[0]["out"]))
    assert float((pending.total().cpu().double() - sum(plain.hyper_step(X, sets[0], "", lambda u: y.double()))).abs().max()) < 1e-4
    got = kernels.streams_norm(streams, w.cuda(), groups, eps, dtype, update=pending, read=f32(sets[1]["in"]))
    X = plain.hyper_step(X, sets[0], "", lambda u: y.double())
    assert float((got.cpu().double() - normed(X, sets[1]["in"])).abs().max()) < tol * 3
    assert float((streams.cpu().double() - torch.stack(X, 1)).abs().max()) < 1e-4
    # a shared expert's output beside routed experts' outputs still in pieces; only some rows: the streams stay
    pieces = torch.randn(M * k, W, generator=g)
    pair_pos = torch.randperm(M * k, generator=g).int()
    pw = torch.rand(M, k, generator=g)
    summed = (pw.double()[:, :, None] * pieces.double()[pair_pos.long()].view(M, k, W)).sum(1)
    both = kernels.DeltaSum(y.cuda(), kernels.ExpertSum(pieces.cuda(), pair_pos.cuda(), pw.cuda()))
    pending = kernels.StreamsDelta(streams, both, f32(sets[1]["mix"]), f32(sets[1]["out"]))
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    kept = streams.clone()
    got = kernels.streams_norm(streams, w.cuda(), groups, eps, dtype, update=pending, rows=rows.cuda())
    X2 = plain.hyper_step(X, sets[1], "", lambda u: y.double() + summed)
    ones = torch.ones(S, dtype=torch.float64)
    assert torch.equal(streams, kept)
    assert float((got.cpu().double() - normed(X2, ones)[rows.long()]).abs().max()) < tol * 3
    # the same on every row, the pieces alone
    pending = kernels.StreamsDelta(streams, both.b, f32(sets[2]["mix"]), f32(sets[2]["out"]))
    got = kernels.streams_norm(streams, w.cuda(), groups, eps, dtype, update=pending, read=f32(sets[0]["in"]))
    X3 = plain.hyper_step(X, sets[2], "", lambda u: summed)
    assert float((got.cpu().double() - normed(X3, sets[0]["in"])).abs().max()) < tol * 3
    assert float((streams.cpu().double() - torch.stack(X3, 1)).abs().max()) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_mix_clamped_gate_silu_head_gate_softmax_router_and_scaled_embedding(dtype):
    from snowllm_b200.ops import kernels
    g = torch.Generator().manual_seed(7)
    M, W = 9, 100
    tol = 1e-5 if dtype == torch.float32 else 0.03
    a, b = torch.randn(M, W, generator=g) * 3, torch.randn(M, W, generator=g) * 0.01
    wa, wb = ((1 + 0.3 * torch.randn(W, generator=g)).to(dtype) for _ in range(2))
    got = kernels.pair_norm_mix(a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), 0.5, 0.5, 1e-4)
    want = 0.5 * (plain.rms(a.double(), 1e-4) * wa.double() + plain.rms(b.double(), 1e-4) * wb.double())
    assert float((got.cpu().double() - want).abs().max()) < 1e-5
    # the experts' activation: the gate is clamped from above only, the other factor on both sides
    gu = (torch.randn(M, 2 * 24, generator=g) * 3).to(dtype)
    got = kernels.gated_act(gu.cuda(), "swish_clamp", limit=1.3)
    gate, up = gu[:, :24].double().clamp(max=1.3), gu[:, 24:].double().clamp(-1.3, 1.3)
    want = gate * torch.sigmoid(plain.SWISH_SLOPE * gate) * (up + 1)
    assert float((got.cpu().double() - want).abs().max()) < tol
    assert float(gu[:, :24].min()) < -1.3 and float(want.min()) < -0.05          # gates far below zero pass
    # heads over their root mean square, times silu of a gate taken from wider rows
    heads, dv = 3, 20
    o = torch.randn(M, heads, dv, generator=g)
    gate = torch.randn(M, 7 + heads * dv, generator=g).to(dtype)
    got = kernels.head_norm_gate(o.cuda(), heads, dv, 1e-2, dtype, gate=gate.cuda(), gate_col=7, gate_act="silu")
    want = plain.rms(o.double(), 1e-2).reshape(M, -1) * plain.silu(gate[:, 7:].double())
    assert float((got.cpu().double() - want).abs().max()) < tol
    wt = (1 + 0.3 * torch.randn(dv, generator=g)).to(dtype)
    got = kernels.head_norm_gate(o.cuda(), heads, dv, 1e-2, dtype, weight=wt.repeat(heads).cuda())
    assert float((got.cpu().double() - (plain.rms(o.double(), 1e-2) * wt.double()).reshape(M, -1)).abs().max()) < tol
    # the router: a softmax over all experts, the largest picked, their scores as they are
    for rows, E, k in ((5, 7, 3), (100, 4, 4), (70, 16, 1)):
        x = torch.randn(rows, 32, generator=g).to(dtype)
        rw = (torch.randn(E, 32, generator=g) * 0.5).to(dtype)
        s = torch.softmax(x.double() @ rw.double().T, -1)
        for route in (kernels.moe_route, lambda *a: kernels.moe_route_sort(*a)[:2]):
            ids, wts = route(x.cuda(), rw.cuda(), None, k, False, 1.0, "softmax")
            picked = torch.gather(s, 1, ids.cpu().long())
            assert float((wts.cpu().double() - picked).abs().max()) < (1e-5 if dtype == torch.float32 else 0.02)
            assert float((picked.sum(-1) - s.topk(k).values.sum(-1)).abs().max()) < (1e-6 if dtype == torch.float32 else 0.02)
            assert all(len(set(r)) == k for r in ids.cpu().tolist())
    # the embedding: rows times a constant, in float
    table = torch.randn(30, 24, generator=g).to(dtype)
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32)
    got = kernels.embedding(ids.cuda(), table.cuda(), scale=2.5)
    assert torch.equal(got.cpu(), table[ids.long()].float() * 2.5)


def clamped_swish(g, u, limit):
    g = g.clamp(max=limit)
    return g * torch.sigmoid(plain.SWISH_SLOPE * g) * (u.clamp(-limit, limit) + 1.0)


@pytest.mark.parametrize("rows", [3, 130, 4300])
@pytest.mark.parametrize("limit", [0.75, 2.3])
def test_products_clamp_and_gate_at_their_store(rows, limit):
    """The few-rows product, the tcgen05 product and the product on pairs of SMs with the clamped swish, plain
    and grouped, against float64 products of the same bfloat16 operands; a limit that many values exceed, and
    one whose bits do not end in zeros."""
    from snowllm_b200.ops import grouped_linear_glu, interleave_gate_up, linear_glu
    g = torch.Generator().manual_seed(rows)
    K, inter, groups = 64, 40, 3
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    gate = (torch.randn(groups, inter, K, generator=g) * 0.3).to(torch.bfloat16)
    up = (torch.randn(groups, inter, K, generator=g) * 0.3).to(torch.bfloat16)
    got = linear_glu(x.cuda(), interleave_gate_up(gate[0], up[0]).cuda(), True, "swish_clamp", limit)
    want = clamped_swish(x.double() @ gate[0].double().T, x.double() @ up[0].double().T, limit)
    assert got.shape == (rows, inter)
    assert bool(((got.cpu().double() - want).abs() <= 0.008 * want.abs() + 2e-3).all())     # one bfloat16 rounding
    assert cases.relative_error(got.cpu(), want) < 0.004
    # rows in group order, unequal groups, one of them empty when there are few rows
    cuts = [0, rows // 2, rows // 2, rows] if rows < 10 else [0, rows // 5, rows // 2, rows]
    offsets = torch.tensor(cuts, dtype=torch.int32).cuda()
    got = grouped_linear_glu(x.cuda(), interleave_gate_up(gate, up).cuda(), offsets, rows, rows, None, 1, True,
                             "swish_clamp", limit)
    want = torch.cat([clamped_swish(x[a:b].double() @ gate[e].double().T, x[a:b].double() @ up[e].double().T, limit)
                      for e, (a, b) in enumerate(zip(cuts[:-1], cuts[1:]))])
    assert bool(((got.cpu().double() - want).abs() <= 0.008 * want.abs() + 2e-3).all())
    assert cases.relative_error(got.cpu(), want) < 0.004


# --- one model with everything: cuts, batches, reuse ------------------------------------------------

@pytest.fixture(scope="module")
def mixed():
    tensors = cases.draw_weights(cases.MIXED, seed=3)
    prompts = {n: cases.tokens_for(cases.MIXED, t, seed=i) for i, (n, t) in
               enumerate((("a", 97), ("b", 41), ("c", 70), ("d", 3)))}
    want = {n: reference(cases.MIXED, tensors, p) for n, p in prompts.items()}
    return tensors, prompts, want


BOUND = {"float32": 2 * F32_TOL, "bfloat16": 2 * BF16_TOL}


def on_engine_picks(tensors, prompts, want, dtype):
    """What the plain implementation gives for each prompt.  For bfloat16 its experts are put on the picks of
    the engine's run of the whole prompt: a near tie between two experts may fall either way after rounding,
    and the row that it falls in would say nothing about the rest."""
    if dtype == "float32":
        return want
    routed = [i for i, l in enumerate(cases.MIXED["layers"]) if l["mlp"] is not None]
    rp = replay(load(cases.MIXED, tensors, dtype), max_tokens=128, requests=1)
    out = {}
    for n, p in prompts.items():
        rp.runner.taps = []
        cases.run_cuts(rp, n, p, [len(p)])
        force = dict(zip(routed, [t.long().sort(-1).values for t in engine_picks(rp)]))
        out[n] = reference(cases.MIXED, tensors, p, picks=force)
    return out


def agree(got, want, dtype, bound=None) -> bool:
    """float32: every row within the bound.  bfloat16: nine rows in ten.  This model's norms run over as few
    as four or eight numbers; where such a group happens to lie near zero, its norm blows the rounding of
    what came before up by orders of magnitude, and that row says nothing about the kernels (float32 does)."""
    bound = BOUND[dtype] if bound is None else bound
    if dtype == "float32":
        return cases.worst_row_error(got, want) < bound
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    rows = torch.sqrt((d * d).mean(-1)) / torch.sqrt((w * w).mean())
    if len(rows) < 8:                                      # too few rows for a share: none far off
        return float(rows.max()) < 5 * bound
    return int((rows >= bound).sum()) <= len(rows) // 10 and float(rows.median()) < bound / 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_every_size_agree_with_the_whole_prompt(mixed, dtype):
    tensors, prompts, want = mixed
    want = on_engine_picks(tensors, {"a": prompts["a"]}, want, dtype)
    rp = replay(load(cases.MIXED, tensors, dtype), max_tokens=128, requests=2)
    toks = prompts["a"]
    whole = cases.run_cuts(rp, "whole", toks, [len(toks)])
    assert agree(whole, want["a"], dtype)
    for sizes in ([2], [3, 16, 1, 29, 2], [16], [17, 1, 1, 1], [64, 2, 2], [1]):
        got = cases.run_cuts(rp, "cut", toks, cases.cuts_of(len(toks), sizes))
        assert agree(got, whole, dtype, 2e-5 if dtype == "float32" else None), sizes
        assert agree(got, want["a"], dtype), sizes
    assert all(p.held() == 0 for p in rp.cache.groups.values()) and rp.cache.slots.free_count == 2


def test_long_portions_walked_in_pieces_agree_with_the_plain_model(mixed, monkeypatch):
    """The memories cut long portions into pieces that blocks of their own walk; with pieces of five rows
    every portion above ten rows goes that way, beside short ones and single tokens that do not."""
    from snowllm_b200.parts import decay_memory
    monkeypatch.setattr(decay_memory, "PIECE_ROWS", 5)
    tensors, prompts, want = mixed
    rp = replay(load(cases.MIXED, tensors, "float32"), max_tokens=256, requests=3)
    for sizes in ([97], [11, 3, 40, 1, 15, 10], [50, 47]):
        got = cases.run_cuts(rp, "cut", prompts["a"], cases.cuts_of(97, sizes))
        assert cases.worst_row_error(got, want["a"]) < BOUND["float32"], sizes
    # two long portions and a single token in one step, then the rest
    a, b, c = prompts["a"], prompts["b"], prompts["c"]            # 97, 41 and 70 tokens
    assert rp.step([{"id": "b", "tokens": b[:40], "want": []}], []) is None
    one = rp.step([{"id": "a", "tokens": a[:60], "want": list(range(60))},
                   {"id": "c", "tokens": c[:33], "want": list(range(33))},
                   {"id": "b", "tokens": b[40:], "want": [0]}], ["b"])
    two = rp.step([{"id": "a", "tokens": a[60:], "want": list(range(37))},
                   {"id": "c", "tokens": c[33:], "want": list(range(37))}], ["a", "c"])
    assert cases.worst_row_error(torch.cat([one[:60], two[:37]]).double(), want["a"]) < BOUND["float32"]
    assert cases.worst_row_error(torch.cat([one[60:93], two[37:]]).double(), want["c"]) < BOUND["float32"]
    assert float((one[93:].double() - want["b"][40:]).abs().max()) < 1e-4 * float(want["b"].abs().max())
    assert all(p.held() == 0 for p in rp.cache.groups.values()) and rp.cache.slots.free_count == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_over_a_small_pool(mixed, dtype):
    """Portions of some requests beside single tokens of others; three slots and few pages, so that slots
    (with the states that earlier requests left in them) and pages are freed and used again; every request's
    logits equal those of its run alone."""
    tensors, prompts, want = mixed
    want = on_engine_picks(tensors, prompts, want, dtype)
    rp = replay(load(cases.MIXED, tensors, dtype), max_tokens=192, requests=3)
    plan = {"a": cases.cuts_of(97, [30, 1, 1, 2, 40, 1]), "b": cases.cuts_of(41, [1, 5, 1, 1, 20]),
            "c": cases.cuts_of(70, [2, 2, 1, 64, 1]), "d": [1, 2]}
    got = {n: [] for n in prompts}
    at = {n: 0 for n in prompts}
    turn = {n: 0 for n in prompts}
    live, waiting, steps = ["a", "b", "d"], ["c"], 0         # d ends early, c takes its slot and pages
    while live:
        entries, ends = [], []
        for n in list(live):
            if steps % 3 == 2 and n == "b" and turn[n] < len(plan[n]) - 1 and len(live) > 1:
                continue                                 # a request may sit out a step
            size = plan[n][turn[n]]
            entries.append({"id": n, "tokens": prompts[n][at[n]:at[n] + size], "want": list(range(size))})
            at[n] += size
            turn[n] += 1
            if turn[n] == len(plan[n]):
                ends.append(n)
        logits = rp.step(entries, ends)
        row = 0
        for e in entries:
            got[e["id"]].append(logits[row:row + len(e["tokens"])].double())
            row += len(e["tokens"])
        for n in ends:
            live.remove(n)
            if waiting:
                live.append(waiting.pop(0))
        steps += 1
    for n in prompts:
        assert at[n] == len(prompts[n])
        assert agree(torch.cat(got[n], 0), want[n], dtype), n
    assert all(p.held() == 0 for p in rp.cache.groups.values()) and rp.cache.slots.free_count == 3


def test_long_decoding_past_every_block_page_and_chunk(mixed):
    tensors, _, _ = mixed
    toks = cases.tokens_for(cases.MIXED, 560, seed=9)
    want = reference(cases.MIXED, tensors, toks)
    rp = replay(load(cases.MIXED, tensors, "float32"), max_tokens=64, requests=1, page_size=8)
    got = cases.run_cuts(rp, "long", toks, [20] + [1] * 540)      # block-local layers give their pages back
    assert cases.worst_row_error(got, want) < F32_TOL * 2
    assert all(p.held() == 0 for p in rp.cache.groups.values())


def test_a_token_just_before_the_blocks_in_reach_does_not_matter():
    """Attention alone passes tokens on (the memories' output weights are zero): the last token's logits keep
    their bits when the token one before the chained blocks changes, and move as the plain implementation
    says when the first token inside changes; in a prompt's portion and decoded alone."""
    cfg = cases.config([cases.pair_layer(chunk=9, mlp=None), cases.pair_layer(heads=2, kv_heads=1, chunk=7)])
    tensors = cases.draw_weights(cfg, seed=11)
    for name in tensors:
        if name.endswith("right.out"):
            tensors[name] = torch.zeros_like(tensors[name])
    toks = cases.tokens_for(cfg, 48)
    # row 47 reads 42..47 in the second layer; row 42 reads 36..42 in the first
    rp = replay(load(cfg, tensors, "float32"), max_tokens=64, requests=1, page_size=8)
    for cuts in ([48], [40] + [1] * 8, [37, 7, 2, 2]):
        base = cases.run_cuts(rp, "x", toks, cuts)[-1]
        beyond = list(toks)
        beyond[35] = (toks[35] + 1) % cfg["vocab"]
        assert torch.equal(cases.run_cuts(rp, "x", beyond, cuts)[-1], base)
        inside = list(toks)
        inside[36] = (toks[36] + 1) % cfg["vocab"]
        moved = cases.run_cuts(rp, "x", inside, cuts)[-1]
        want = reference(cfg, tensors, inside)[-1] - reference(cfg, tensors, toks)[-1]
        assert float(want.abs().max()) > 1e-4
        assert float(((moved - base) - want).abs().max()) < 2e-5


def test_a_memory_never_forgets_what_a_decay_of_one_keeps():
    """A retention head with decay 1 and one far token whose key stands out: hundreds of tokens later, in a
    prompt and decoded, the logits still depend on it exactly as the plain implementation says."""
    cfg = cases.config([cases.pair_layer(chunk=16, r_heads=2, r_dim=8, r_vdim=8, decay=(1.0, 0.96875), rot_dims=4, mlp=None)])
    tensors = cases.draw_weights(cfg, seed=12)
    toks = cases.tokens_for(cfg, 330)
    other = list(toks)
    other[2] = (toks[2] + 7) % cfg["vocab"]
    want = reference(cfg, tensors, other)[-1] - reference(cfg, tensors, toks)[-1]
    assert float(want.abs().max()) > 1e-3
    rp = replay(load(cfg, tensors, "float32"), max_tokens=384, requests=1, page_size=16)
    for cuts in ([330], [290] + [1] * 40):
        moved = cases.run_cuts(rp, "x", other, cuts)[-1] - cases.run_cuts(rp, "x", toks, cuts)[-1]
        assert float((moved - want).abs().max()) < 5e-5


# --- through the loader, the scheduler and the sampler ----------------------------------------------

@pytest.mark.parametrize("dtype,eager", [("float32", False), ("float32", True), ("bfloat16", False)])
def test_greedy_generation_through_the_engine(tmp_path, mixed, dtype, eager):
    import snowllm_b200
    from snowllm_b200.engine import Engine, SamplingParams
    tensors, prompts, _ = mixed
    cases.write_folder(tmp_path, cases.MIXED, tensors)
    model = snowllm_b200.load(tmp_path, dtype, "cuda")
    engine = Engine(model, max_num_seqs=2, max_model_len=256, prefill_chunk=24, page_size=16, enforce_eager=eager)
    asked = [prompts["b"], prompts["d"], prompts["c"][:30]]
    outs = engine.generate(asked, SamplingParams(temperature=0, max_new_tokens=40))
    # float32 against the plain implementation; bfloat16 (whose rounding a small norm group can blow up)
    # against the step function fed the same tokens whole: scheduler, portions and captured steps add nothing
    slack = 1e-4 if dtype == "float32" else 0.15
    rp = replay(load(cases.MIXED, tensors, dtype), max_tokens=128, requests=1) if dtype != "float32" else None
    for p, o in zip(asked, outs):
        assert len(o) == 40
        logits = reference(cases.MIXED, tensors, p + o) if rp is None else cases.run_cuts(rp, "r", p + o, [len(p + o)])
        for i, tok in enumerate(o):
            row = logits[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= slack, (dtype, i, tok, int(row.argmax()))
    if not eager:
        assert engine.runner.graph_replays > 0


def test_command_line_generates_with_the_design(tmp_path, mixed, capsys):
    import json

    from snowllm_b200 import cli
    tensors, prompts, _ = mixed
    cases.write_folder(tmp_path, cases.MIXED, tensors)
    prompt = prompts["b"][:20]
    rc = cli.main([str(tmp_path), "--prompt-ids", ",".join(map(str, prompt)), "--default-max-tokens", "12",
                   "--dtype", "float32", "--max-model-len", "256", "--kv-block-size", "16", "--max-num-seqs", "2"])
    assert rc == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[0])
    assert line["prompt_tokens"] == 20 and len(line["tokens"]) == 12 and line["finish_reason"] == "length"
    logits = reference(cases.MIXED, tensors, prompt + line["tokens"])
    for i, tok in enumerate(line["tokens"]):
        row = logits[len(prompt) - 1 + i]
        assert float(row.max() - row[tok]) <= 1e-4
