"""The kernels that the Narasun parts add, each against a few lines of PyTorch in float64: the sink in every
attention kernel, the query temperature, the residual sum with its norm, the token shift, the decay network,
the capped gates, the two scans (also in portions, which must give the same bits as one pass), and the
routed feed-forward with several experts per token."""
import math

import pytest
import torch

import plain_narasun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype).to(DEV)


def close(got, ref, tol):
    ref = ref.double().cpu()
    err = float((got.double().cpu() - ref).abs().max() / ref.abs().max())
    assert err < tol, err


@pytest.mark.parametrize("dtype,hd,T,tol", [(torch.float32, 24, 150, 1e-5), (torch.bfloat16, 48, 300, 2e-2),
                                              (torch.bfloat16, 64, 1200, 2e-2), (torch.bfloat16, 128, 900, 2e-2)])
def test_prefill_attention_with_a_sink(dtype, hd, T, tol):
    """simt (float32), mma.sync (bfloat16, short) and tcgen05 (bfloat16, heads of 64 and 128, long) with a sink;
    one far key is made to carry the last query's weight, and one head's sink to outweigh its scores."""
    from catena_models_b200 import kernels
    from catena_models_b200.engine.runtime import Runtime

    QH, KVH = 4, 2
    rt = Runtime(dtype, DEV)
    buf = rnd(T, (QH + 2 * KVH) * hd, seed=1, dtype=dtype)
    q, k, v = buf[:, :QH * hd], buf[:, QH * hd:(QH + KVH) * hd], buf[:, (QH + KVH) * hd:]
    k[3] *= 3.0                                       # a key far from the last queries that several of them pick
    sink = torch.tensor([4.0, -2.0, 0.0, 9.0], device=DEV)
    scale = 0.5 / math.sqrt(hd)
    seq_start = torch.tensor([0, T - 40, T], dtype=torch.int32, device=DEV)

    class B:
        pass
    batch = B()
    batch.seq_start, batch.B, batch.max_len = seq_start, 2, T - 40
    ctx = torch.empty((T, QH * hd), dtype=dtype, device=DEV)
    rt.attention_prefill(ctx, q, k, v, None, batch, QH, KVH, hd, 0, scale, sink=sink)
    rt.check_errors()
    qd, kd, vd = (x.double().cpu() for x in (q, k, v))
    for s0, s1 in ((0, T - 40), (T - 40, T)):
        ref = plain.sink_attention_heads(qd[s0:s1].view(-1, QH, hd), kd[s0:s1].view(-1, KVH, hd),
                                         vd[s0:s1].view(-1, KVH, hd), sink.double().cpu(), scale, 0.0, 0)
        close(ctx[s0:s1], ref.reshape(s1 - s0, -1), tol)


def test_query_temperature():
    from catena_models_b200 import kernels

    T, QH, KVH, hd = 70, 3, 1, 16
    buf = rnd(T, (QH + 2 * KVH) * hd, seed=2)
    before = buf.clone()
    pos = torch.arange(5, 5 + T, dtype=torch.int32, device=DEV)
    zeros = torch.zeros(T, dtype=torch.int32, device=DEV)
    one = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.qk_prepare(buf, None, None, None, pos, zeros, one, one + 200, None, 0, None, 0, QH, KVH, hd, 0.0, q_temp=(0.4, 8))
    temp = 1.0 + 0.4 * torch.log(torch.div(pos.cpu() + 1, 8, rounding_mode="floor").double() + 1.0)
    close(buf[:, :QH * hd], before[:, :QH * hd].double().cpu() * temp[:, None], 1e-6)
    assert torch.equal(buf[:, QH * hd:], before[:, QH * hd:])          # keys and values stay


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual_sum_and_norm(dtype):
    from catena_models_b200 import kernels

    rows, H = 9, 72
    h = rnd(rows, H, seed=3)
    a, b = rnd(rows, H, seed=4, dtype=dtype), rnd(rows * 3, H, seed=5)
    bias, w = rnd(H, seed=6), rnd(H, seed=7)
    ref = h.double() + (0.7 * a.double() + 1.3 * b.double().view(rows, 3, H).sum(1)) + bias.double()
    n = torch.empty((rows, H), dtype=dtype, device=DEV)
    order = torch.randperm(rows * 3, device=DEV).to(torch.int32)
    shuffled = torch.empty_like(b)
    shuffled[order.long()] = b
    kernels.residual_add_norm(h, kernels.Terms([(a, 0.7, 1), (shuffled, 1.3, 3, order)]), n, w, 1e-5, bias)
    close(h, ref, 1e-6)
    close(n, plain.rms_unit(ref, 1e-5) * w.double(), 1e-6 if dtype == torch.float32 else 1e-2)
    y = torch.empty((rows, H), dtype=dtype, device=DEV)
    kernels.norm_f32in(y, h, w, 1e-5)
    assert torch.equal(y, n)
    both = torch.empty((rows, 2 * H), dtype=dtype, device=DEV)
    kernels.concat_cast(both, h, ref.float())
    assert torch.equal(both, torch.cat([h, ref.float()], 1).to(dtype))


def _scan_inputs(T, H, D, DV, seed):
    q, k = rnd(T, H * D, seed=seed), rnd(T, H * D, seed=seed + 1, std=0.5)
    v, g = rnd(T, H * DV, seed=seed + 2), rnd(T, H * DV, seed=seed + 3)
    return q, k, v, g


@pytest.mark.parametrize("H,D,DV", [(2, 24, 40), (1, 8, 8), (3, 64, 16), (2, 40, 300)])
def test_matrix_memory_scan(H, D, DV):
    """Against the plain recurrence; in portions the same bits as in one pass; the state of another slot untouched."""
    from catena_models_b200 import kernels

    T, eps = 50, 1e-5
    q, k, v, g = _scan_inputs(T, H, D, DV, 10)
    gates = torch.cat([rnd(T, H, seed=14, std=3.0), -torch.rand(T, H, device=DEV) * 0.3], 1).contiguous()
    nw = rnd(H * DV, seed=15)
    per = H * (D * DV + D + 1)
    state = torch.zeros((3, per), device=DEV)
    state[2] = 7.0
    slot = torch.tensor([1], dtype=torch.int32, device=DEV)
    out = torch.empty((T, H * DV), device=DEV)
    run = lambda o, a, b: kernels.matrix_scan("memory", o[a:b], q[a:b], k[a:b], v[a:b], g[a:b], gates[a:b], None, nw, state, 0,
                                              torch.tensor([0, b - a], dtype=torch.int32, device=DEV), slot, 1, H, D, DV,
                                              D ** -0.5, eps)
    run(out, 0, T)
    # plain: S, n, m per head
    qd, kd, vd, gd, gt = (x.double().cpu() for x in (q, k, v, g, gates))
    S, n, m = torch.zeros(H, D, DV, dtype=torch.float64), torch.zeros(H, D, dtype=torch.float64), torch.zeros(H, dtype=torch.float64)
    ref = torch.zeros(T, H, DV, dtype=torch.float64)
    for t in range(T):
        qq, kk, vv = qd[t].view(H, D) * D ** -0.5, kd[t].view(H, D), vd[t].view(H, DV)
        i_, f_ = gt[t, :H], gt[t, H:]
        m2 = torch.maximum(f_ + m, i_)
        a_, b_ = torch.exp(f_ + m - m2), torch.exp(i_ - m2)
        S = a_[:, None, None] * S + b_[:, None, None] * kk[:, :, None] * vv[:, None, :]
        n = a_[:, None] * n + b_[:, None] * kk
        m = m2
        den = torch.maximum((n * qq).sum(-1).abs(), torch.exp(-m)) + 1e-6
        ref[t] = torch.einsum("hkv,hk->hv", S, qq) / den[:, None]
    ref = plain.rms_unit(ref, eps).reshape(T, -1) * nw.double().cpu() * torch.sigmoid(gd)
    close(out, ref, 2e-5)
    assert bool((state[2] == 7.0).all()) and bool((state[0] == 0.0).all())
    final = state[1].clone()
    state[1] = 0.0
    parts = torch.empty_like(out)
    for a, b in ((0, 2), (2, 3), (3, 31), (31, T)):
        run(parts, a, b)
    assert torch.equal(parts, out) and torch.equal(state[1], final)


@pytest.mark.parametrize("H,D", [(2, 16), (1, 40), (3, 64)])
def test_decay_scan(H, D):
    from catena_models_b200 import kernels

    T, W, eps = 45, 24, 1e-6
    q, k, v, g = _scan_inputs(T, H, D, D, 20)
    decay = torch.rand(T, H * D, device=DEV) * 0.8 + 0.19
    u, nw = rnd(H, D, seed=24, std=0.5), rnd(H * D, seed=25)
    x = rnd(T, W, seed=26)
    state = torch.zeros((2, W + H * D * D), device=DEV)
    slot = torch.tensor([1], dtype=torch.int32, device=DEV)
    out = torch.empty((T, H * D), device=DEV)
    run = lambda o, a, b: kernels.matrix_scan("decay", o[a:b], q[a:b], k[a:b], v[a:b], g[a:b], decay[a:b], u, nw, state, W,
                                              torch.tensor([0, b - a], dtype=torch.int32, device=DEV), slot, 1, H, D, D, 1.0,
                                              eps, shift_src=x[a:b])
    run(out, 0, T)
    qd, kd, vd, gd, wd = (t.double().cpu() for t in (q, k, v, g, decay))
    S = torch.zeros(H, D, D, dtype=torch.float64)
    ref = torch.zeros(T, H, D, dtype=torch.float64)
    for t in range(T):
        kv = kd[t].view(H, D)[:, :, None] * vd[t].view(H, D)[:, None, :]
        ref[t] = torch.einsum("hkv,hk->hv", S + u.double().cpu()[:, :, None] * kv, qd[t].view(H, D))
        S = wd[t].view(H, D)[:, :, None] * S + kv
    ref = plain.rms_unit(ref, eps).reshape(T, -1) * nw.double().cpu() * plain.silu(gd)
    close(out, ref, 2e-5)
    assert torch.equal(state[1, :W], x[-1]) and bool((state[0] == 0).all())       # the last input is kept for the next step
    final = state[1].clone()
    state[1] = 0.0
    parts = torch.empty_like(out)
    for a, b in ((0, 1), (1, 3), (3, 40), (40, T)):
        run(parts, a, b)
    assert torch.equal(parts, out) and torch.equal(state[1], final)


def test_token_shift_decay_network_and_gates():
    from catena_models_b200 import kernels

    T, W, R, C, H = 11, 40, 6, 48, 3
    h, mu = rnd(T, W, seed=30), torch.rand(5, W, device=DEV)
    state = rnd(2, W + 5, seed=31)
    # two sequences: rows 0..6 go on at position 3 (their previous input is in the state), rows 7..10 likewise at 9
    tok_seq = torch.tensor([0] * 7 + [1] * 4, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(list(range(3, 10)) + list(range(9, 13)), dtype=torch.int32, device=DEV)
    pos0 = torch.tensor([3, 9], dtype=torch.int32, device=DEV)
    slot = torch.tensor([1, 0], dtype=torch.int32, device=DEV)
    out = torch.empty((5, T, W), device=DEV)
    kernels.shift_mix(out, h, mu, state, tok_seq, tok_pos, pos0, slot)
    prev = torch.cat([state[1, :W][None], h[:6], state[0, :W][None], h[7:10]])
    close(out, h.double()[None] + (prev.double() - h.double())[None] * mu.double()[:, None], 1e-6)
    w1, w2, w0 = rnd(R, W, seed=32, std=0.3), rnd(C, R, seed=33), rnd(C, seed=34)
    dec = torch.empty((T, C), device=DEV)
    kernels.lowrank_decay(dec, h, w1, w2.t().contiguous(), w0)
    close(dec, torch.exp(-torch.exp(torch.tanh(h.double() @ w1.double().T) @ w2.double().T + w0.double())), 1e-5)
    wg, bias, cap = rnd(2 * H, W, seed=35), rnd(2 * H, seed=36), 4.0
    gates = torch.empty((T, 2 * H), device=DEV)
    kernels.capped_gates(gates, h, wg, bias, cap)
    z = cap * torch.tanh((h.double() @ wg.double().T + bias.double()) / cap)
    close(gates, torch.cat([z[:, :H], torch.nn.functional.logsigmoid(z[:, H:])], 1), 1e-5)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("T,E,top", [(70, 7, 3), (5, 3, 1), (300, 40, 2)])
def test_routed_feed_forward(dtype, tol, T, E, top):
    """Router, ordering by expert and both grouped products against a loop over tokens; rows of padding are skipped."""
    from catena_models_b200 import kernels

    W, F = 40, 24
    h = rnd(T, W, seed=40, dtype=dtype)
    wr = rnd(E, W, seed=41, std=0.5, dtype=dtype)
    w_up, w_down = rnd(E, 2 * F, W, seed=42, std=0.2, dtype=dtype), rnd(E, W, F, seed=43, std=0.2, dtype=dtype)
    tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    tok_seq[T - 1] = -1                                                     # a row of padding
    P = T * top
    tiles = kernels.moe_max_tiles(P, E)
    rows = tiles * kernels.MOE_TILE_SIMT
    ids, wts = torch.empty(P, dtype=torch.int32, device=DEV), torch.empty(P, device=DEV)
    perm, dest = torch.empty(rows, dtype=torch.int32, device=DEV), torch.empty(P, dtype=torch.int32, device=DEV)
    work = torch.empty(kernels.moe_work_size(P, E), dtype=torch.int32, device=DEV)
    kernels.moe_route(ids, wts, perm, dest, work, h, wr, tok_seq, top)
    a = torch.empty((rows, F), dtype=dtype, device=DEV)
    kernels.moe_grouped(a, h, w_up, work, perm, wts, top, tiles, up=True, apply_weight=True)
    y = torch.zeros((rows, W), device=DEV)
    kernels.moe_grouped(y, a, w_down, work, perm, wts, top, tiles, up=False, apply_weight=False)
    where = dest.view(T, top)[:T - 1].long()
    got = y[where].sum(1)
    if dtype == torch.bfloat16:
        # the same rows through the grouped tcgen05 product (row tiles of 128)
        big = kernels.MOE_TILE_TC
        tiles2 = kernels.moe_max_tiles(P, E, big)
        rows2 = tiles2 * big
        perm2, dest2 = torch.empty(rows2, dtype=torch.int32, device=DEV), torch.empty(P, dtype=torch.int32, device=DEV)
        work2 = torch.empty(kernels.moe_work_size(P, E, big), dtype=torch.int32, device=DEV)
        ids2, wts2 = torch.empty_like(ids), torch.empty_like(wts)
        kernels.moe_route(ids2, wts2, perm2, dest2, work2, h, wr, tok_seq, top, tile_rows=big)
        assert torch.equal(ids2, ids)
        groups = kernels.moe_tile_group(work2, P, E, big)
        xs = torch.empty((rows2, W), dtype=dtype, device=DEV)
        kernels.moe_gather(xs, h, dest2, wts2, top, True)
        a2 = torch.empty((rows2, F), dtype=dtype, device=DEV)
        kernels.gemm_tc_grouped(a2, xs, w_up, groups, swiglu=True, block_n=128)
        y2 = torch.empty((rows2, W), device=DEV)
        kernels.gemm_tc_grouped(y2, a2, w_down, groups, block_n=128)
        got2 = y2[dest2.view(T, top)[:T - 1].long()].sum(1)
        assert float((got2 - got).abs().max() / got.abs().max()) < 2e-2
        got = got2
    hd = h.double().cpu()
    s = torch.sigmoid(hd @ wr.double().cpu().T)
    rdt = (lambda x: x.to(dtype).double())
    ref = torch.zeros(T - 1, W, dtype=torch.float64)
    chosen = ids.view(T, top).cpu()
    for t in range(T - 1):
        order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        if dtype == torch.float32:
            assert order == chosen[t].tolist()
        for e in chosen[t].tolist():
            x = rdt(s[t, e] * hd[t])
            g, u = w_up[e, :F].double().cpu() @ x, w_up[e, F:].double().cpu() @ x
            ref[t] += w_down[e].double().cpu() @ rdt(plain.silu(g) * u)
    close(got, ref, tol)
    assert bool((ids.view(T, top)[T - 1] == -1).all()) and bool((dest.view(T, top)[T - 1] == -1).all())


def test_routed_feed_forward_paths_agree_in_a_model(tmp_path):
    """The grouped tcgen05 product and the CUDA-core grouped products give a bfloat16 model the same logits up to
    rounding (a model whose two experts are both chosen for every token, so that no choice can fall differently)."""
    import tiny_narasun as tiny
    from catena_models_b200.api import Model

    cfg = dict(architecture="Narasun", vocab=64, width=64, norm=dict(eps=1e-6), loop=None, layers=[
        tiny.mlstm(2, 16, 16, 8.0, tiny.moe(40, 2, 2))])
    folder = tiny.make_folder(tmp_path, "both", seed=5, config=cfg)
    tokens = tiny.prompt(150, 64, 9)
    out = []
    for tensor_cores in (True, False):
        model = Model.load(folder, dtype="bfloat16", max_tokens=512)
        model.decoder.rt.grouped_tensor_cores = tensor_cores
        (slot,) = model.engine.admit(1)
        out.append(model.engine.step([slot], [tokens], [list(range(150))]).float().cpu())
        model.engine.check_errors()
    err = (out[0] - out[1]).abs().amax(-1) / out[1].abs().amax(-1)
    assert float(err.median()) < 0.01 and float(err.max()) < 0.06
