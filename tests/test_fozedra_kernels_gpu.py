"""The kernels that the Fozedra decoder added, each against the plain statement of its mechanism
(plain_fozedra.py, float64): the dynamic tanh alone and behind a residual sum, the squared ReLU, the scan with
one constant decay per head (whole, in portions, several sequences, a slot used again), the taps with rotation
and cache write (whole, portions down to one token, unequal sequences), and the difference of two softmax maps
over the paged cache in both of its forms, with keys placed just inside and just outside the window and the
kept first tokens so that a mask that is one token off changes the result beyond any tolerance."""
import types

import pytest
import torch

import plain_fozedra as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _close(got, ref, tol):
    ref = ref.to(torch.float64).cpu()
    err = (got.to(torch.float64).cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-9)
    assert float(err) < tol, float(err)


def _batch(lengths, starts, slots):
    """What the kernels read of a step: sequences of `lengths` new tokens that stand at `starts`."""
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tok_seq, tok_pos, seq_start = [], [], [0]
    for b, (n, p) in enumerate(zip(lengths, starts)):
        tok_seq += [b] * n
        tok_pos += list(range(p, p + n))
        seq_start.append(seq_start[-1] + n)
    return types.SimpleNamespace(tok_seq=i32(tok_seq), tok_pos=i32(tok_pos), seq_start=i32(seq_start), seq_pos0=i32(starts),
                                 seq_slot=i32(slots), B=len(lengths), T=sum(lengths), max_len=max(lengths))


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 2e-6), (torch.bfloat16, 6e-3)])
def test_dynamic_tanh_alone_and_behind_a_sum(dtype, tol):
    from catena_models_b200 import kernels

    g = torch.Generator().manual_seed(1)
    rows, W = 37, 52
    x = torch.randn(rows, W, generator=g) * 2
    w, b, alpha = 1 + 0.1 * torch.randn(W, generator=g), 0.3 * torch.randn(W, generator=g), torch.tensor([0.61])
    ref = plain.dyt(x.double(), alpha.double(), w.double(), b.double())
    y = torch.empty(rows, W, dtype=dtype, device=DEV)
    kernels.norm_f32in(y, x.to(DEV), w.to(DEV), 0.0, dyt=(alpha.to(DEV), b.to(DEV)))
    _close(y, ref, tol)
    # h += 0.5 * term, then the dynamic tanh of the sum in the same launch
    term = torch.randn(rows, W, generator=g)
    h = x.to(DEV).clone()
    n_out = torch.empty(rows, W, dtype=dtype, device=DEV)
    kernels.residual_add_norm(h, kernels.Terms([(term.to(DEV), 0.5, 1)]), n_out, w.to(DEV), 0.0, dyt=(alpha.to(DEV), b.to(DEV)))
    total = x.double() + 0.5 * term.double()
    _close(h, total, 1e-6)
    _close(n_out, plain.dyt(total, alpha.double(), w.double(), b.double()), tol)


def test_squared_relu():
    from catena_models_b200 import kernels

    x = torch.randn(33, 19, generator=torch.Generator().manual_seed(2))
    for dtype in (torch.float32, torch.bfloat16):
        a = x.to(DEV, dtype).contiguous()
        ref = torch.relu(a.double().cpu()) ** 2
        kernels.relu2_inplace(a)
        _close(a, ref, 1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("H, D, DV", [(2, 16, 24), (1, 12, 20), (3, 4, 12), (4, 64, 32), (2, 7, 9)])
def test_constant_decay_scan_whole_portions_and_slots(H, D, DV, chunked):
    """`chunked`: the prompt form that regroups the sums into chunks of 64 rows, against the same plain statement."""
    from catena_models_b200 import kernels

    g = torch.Generator().manual_seed(3)
    lengths = [45, 1, 70] if not chunked else [200, 1, 129]
    T = sum(lengths)
    q, k, v, gate = (torch.randn(T, n, generator=g) for n in (H * D, H * D, H * DV, H * DV))
    decay = torch.tensor([0.6 + 0.39 * (i + 1) / H for i in range(H)])
    norm_w = 1 + 0.1 * torch.randn(H * DV, generator=g)
    eps = 1e-5

    def reference(lo, hi):
        s = plain.silu
        o = plain.lightning_heads(s(q[lo:hi].double()).view(-1, H, D), s(k[lo:hi].double()).view(-1, H, D),
                                  s(v[lo:hi].double()).view(-1, H, DV), decay.double()).reshape(hi - lo, H * DV)
        return plain.rms_unit(o, eps) * norm_w.double() * torch.sigmoid(gate[lo:hi].double())

    bounds = [0, lengths[0], lengths[0] + 1, T]
    ref = torch.cat([reference(bounds[i], bounds[i + 1]) for i in range(3)])
    state = torch.full((5, H * D * DV), float("nan"), device=DEV)
    dq, dk, dv, dg = (t.to(DEV) for t in (q, k, v, gate))

    def run(cuts, slots):
        """Every sequence in steps of cuts[i] rows (all sequences in one launch per step)."""
        kernels.zero_slots(state.view(1, 5, -1), slots)
        out = torch.empty(T, H * DV, device=DEV)
        at = [0, 0, 0]
        while any(at[i] < lengths[i] for i in range(3)):
            rows, lens, sl = [], [], []
            for i in range(3):
                n = min(cuts[i], lengths[i] - at[i])
                if n > 0:
                    rows += list(range(bounds[i] + at[i], bounds[i] + at[i] + n))
                    lens.append(n)
                    sl.append(slots[i])
                    at[i] += n
            idx = torch.tensor(rows, device=DEV)
            b = _batch(lens, [0] * len(lens), sl)
            o = torch.empty(len(rows), H * DV, device=DEV)
            scratch = None
            if chunked:
                scratch = torch.full((kernels.lightning_scratch_floats(b.B, b.max_len, H, D, DV),), float("nan"), device=DEV)
            kernels.matrix_scan("constant", o, dq[idx], dk[idx], dv[idx], dg[idx], decay.to(DEV), None, norm_w.to(DEV), state, 0,
                                b.seq_start, b.seq_slot, b.B, H, D, DV, 1.0, eps, qkv_silu=True, norm_all_heads=True,
                                chunk_scratch=scratch, max_len=b.max_len)
            out[idx] = o
        return out

    _close(run([1000, 1000, 1000], [0, 1, 2]), ref, 2e-5)
    _close(run([7, 1, 33], [4, 2, 0]), ref, 2e-5)            # portions; the slots of before, used again
    _close(run([65, 1, 64] if chunked else [2, 1, 1], [1, 0, 3]), ref, 2e-5)     # chunk borders; or two tokens and token by token


def _taps_case(seed, H, G, D, DV, K, rot, lengths):
    g = torch.Generator().manual_seed(seed)
    QC, KC, VC = H * 2 * D, G * 2 * D, G * DV
    C = QC + KC + VC
    return dict(H=H, G=G, D=D, DV=DV, K=K, rot=rot, QC=QC, KC=KC, VC=VC, C=C, lengths=lengths,
                proj=[torch.randn(n, C + H, generator=g) for n in lengths], bias=0.3 * torch.randn(C, generator=g),
                taps=0.6 * torch.randn(C, K, generator=g), rates=[0.9 ** i for i in range(rot // 2)], mag=1.07)


def _taps_reference(c, i):
    u = c["proj"][i][:, :c["C"]].double() + c["bias"].double()
    y = plain.causal_taps(u, c["taps"].double())
    n = y.shape[0]
    q = plain.rotate_front(y[:, :c["QC"]].reshape(n, -1, c["D"]), 0, c["rot"], c["rates"], c["mag"]).reshape(n, -1)
    k = plain.rotate_front(y[:, c["QC"]:c["QC"] + c["KC"]].reshape(n, -1, c["D"]), 0, c["rot"], c["rates"], c["mag"]).reshape(n, -1)
    return q, k, y[:, c["QC"] + c["KC"]:]


def _run_taps(c, cuts, slots, dtype=torch.float32, pool=None, state=None):
    """The sequences of case `c` in steps of cuts[i] tokens; returns (queries per sequence, pool, page table)."""
    from catena_models_b200 import kernels

    HDC = -(-max(2 * c["D"], c["DV"]) // 8) * 8
    n_seq = len(c["lengths"])
    pages_per = max(1, -(-max(c["lengths"]) // 64))
    if pool is None:
        pool = torch.full((2, 8 * pages_per, c["G"], 64, HDC), float("nan"), dtype=dtype, device=DEV)
    # pages dealt out in an order of their own, so that a page id is never a sequence's index
    ptab = torch.zeros(8, pages_per, dtype=torch.int32, device=DEV)
    for s in range(8):
        for j in range(pages_per):
            ptab[s, j] = (s * 5 + j * 3) % (8 * pages_per) if pages_per > 1 else (s * 5) % 8
    if pages_per > 1:
        ids = torch.randperm(8 * pages_per, generator=torch.Generator().manual_seed(9)).to(torch.int32).view(8, pages_per)
        ptab.copy_(ids.to(DEV))
    if state is None:
        state = torch.full((8, max(1, c["K"] * c["C"])), float("nan"), device=DEV)
    kernels.zero_slots(state.view(1, 8, -1), slots)
    rate = torch.tensor(c["rates"], dtype=torch.float32, device=DEV) if c["rot"] else None
    qs = [torch.empty(n, c["QC"], dtype=dtype, device=DEV) for n in c["lengths"]]
    at = [0] * n_seq
    while any(at[i] < c["lengths"][i] for i in range(n_seq)):
        rows, lens, starts, sl, who = [], [], [], [], []
        for i in range(n_seq):
            n = min(cuts[i], c["lengths"][i] - at[i])
            if n > 0:
                rows.append(c["proj"][i][at[i]:at[i] + n])
                lens.append(n); starts.append(at[i]); sl.append(slots[i]); who.append(i)
                at[i] += n
        b = _batch(lens, starts, sl)
        proj = torch.cat(rows).to(DEV, dtype)
        q = torch.empty(b.T, c["QC"], dtype=dtype, device=DEV)
        kernels.tap_rotate_store(proj, c["bias"].to(DEV), c["taps"].to(DEV), state, q, b, c["QC"], c["D"], rate, c["mag"],
                                 kv=(pool, pool.shape[1], ptab, c["G"], 2 * c["D"], c["DV"]),
                                 one_token_each=all(n == 1 for n in lens) and all(p > 0 for p in starts))
        o = 0
        for i, n in zip(who, lens):
            qs[i][at[i] - n:at[i]] = q[o:o + n]
            o += n
    return qs, pool, ptab


def _cached(pool, ptab, slot, length, kv, width):
    """[length, G * width]: what the cache holds of a sequence."""
    rows = []
    for p in range(length):
        page = int(ptab[slot, p // 64])
        rows.append(pool[kv, page, :, p % 64, :width].reshape(-1))
    return torch.stack(rows)


@pytest.mark.parametrize("H, G, D, DV, K, rot", [(4, 2, 16, 8, 4, 16), (3, 1, 12, 20, 5, 6), (2, 2, 8, 16, 2, 4), (2, 1, 16, 16, 1, 8),
                                                 (2, 1, 8, 8, 3, 0), (2, 1, 32, 24, 4, 16), (4, 2, 16, 40, 3, 0)])
def test_taps_rotation_and_cache_write(H, G, D, DV, K, rot):
    c = _taps_case(4, H, G, D, DV, K, rot, [70, 3, 530])    # the last one long enough for the form of long steps
    refs = [_taps_reference(c, i) for i in range(3)]
    for cuts, slots in (([1000] * 3, [0, 1, 2]), ([7, 2, 64], [5, 0, 3]), ([1, 1, 1], [2, 6, 1]), ([2, 3, 517], [7, 4, 0])):
        qs, pool, ptab = _run_taps(c, cuts, slots)
        for i, n in enumerate(c["lengths"]):
            _close(qs[i], refs[i][0], 2e-5)
            _close(_cached(pool, ptab, slots[i], n, 0, 2 * D), refs[i][1], 2e-5)
            _close(_cached(pool, ptab, slots[i], n, 1, DV), refs[i][2], 3e-6)
    # bfloat16 rows (the serving engine's): against the same statement on the rounded projections
    for i in range(3):
        c["proj"][i] = c["proj"][i].to(torch.bfloat16).float()
    refs = [_taps_reference(c, i) for i in range(3)]
    for cuts, slots in (([1000] * 3, [0, 1, 2]), ([1, 1, 1], [2, 6, 1])):
        qs, pool, ptab = _run_taps(c, cuts, slots, dtype=torch.bfloat16)
        for i, n in enumerate(c["lengths"]):
            _close(qs[i], refs[i][0], 6e-3)
            _close(_cached(pool, ptab, slots[i], n, 0, 2 * D), refs[i][1], 6e-3)
            _close(_cached(pool, ptab, slots[i], n, 1, DV), refs[i][2], 6e-3)


def _attention_case(seed, H, G, D, DV, T, window, keep, stand_out=None):
    """Random queries, keys and values for one sequence of T tokens; `stand_out` = (query position, key position):
    that query and that key are scaled so that their score dwarfs all others of the query, in both maps."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = torch.randn(T, H, 2, D, generator=g), torch.randn(T, G, 2, D, generator=g), torch.randn(T, G, DV, generator=g)
    if stand_out:
        qi, kj = stand_out
        k[kj] = q[qi, 0:1].expand(G, 2, D) * 3.0          # every key/value head's key points along head 0's query
        q[qi] = q[qi, 0:1] * 3.0
    return q, k, v


def _run_attention(q, k, v, window, keep, scale, lam, out_scale, eps, gate, rows_form, dtype=torch.float32, split=None, shares=1,
                   tensor_cores=False):
    """Through the kernel: keys and values are placed in scattered pages first.  split: the step brings the rows from
    `split` on (the earlier ones are held)."""
    from catena_models_b200 import kernels

    T, H, _, D = q.shape
    G, DV = v.shape[1:]
    HDC = -(-max(2 * D, DV) // 8) * 8
    n_pages = -(-T // 64)
    pool = torch.full((2, 3 * n_pages + 2, G, 64, HDC), float("nan"), dtype=dtype, device=DEV)
    ids = (torch.randperm(3 * n_pages + 2, generator=torch.Generator().manual_seed(5))[:n_pages]).to(torch.int32)
    ptab = torch.full((4, n_pages), -1, dtype=torch.int32, device=DEV)
    ptab[2] = ids.to(DEV)
    for p in range(T):
        pool[0, int(ids[p // 64]), :, p % 64, :2 * D] = k[p].reshape(G, 2 * D).to(DEV, dtype)
        pool[1, int(ids[p // 64]), :, p % 64, :DV] = v[p].to(DEV, dtype)
    first = split or 0
    b = _batch([T - first], [first], [2])
    qq = q[first:].reshape(T - first, -1).to(DEV, dtype).contiguous()
    ctx = torch.empty(T - first, H * DV, dtype=dtype, device=DEV)
    gg = gate[first:].to(DEV, dtype).contiguous() if gate is not None else None
    parts = torch.full(((T - first) * H * shares * (4 + 2 * DV),), float("nan"), device=DEV) if shares > 1 else None
    kernels.diff_attn(ctx, qq, gg, pool, pool.shape[1], ptab, b, H, G, D, DV, window, keep, scale, lam, out_scale, eps, rows_form,
                      parts=parts, splits=shares, tensor_cores=tensor_cores)
    return ctx


@pytest.mark.parametrize("H, G, D, DV, T, window, keep", [
    (4, 2, 16, 8, 150, 9, 3), (3, 1, 12, 20, 200, 70, 0), (2, 2, 8, 16, 90, 5, 11), (4, 1, 16, 24, 140, 64, 32), (8, 2, 12, 20, 100, 30, 5),
    (2, 1, 8, 40, 100, 0, 0), (1, 1, 4, 4, 66, 1, 1), (2, 2, 64, 128, 130, 44, 18)])
def test_two_maps_over_the_cache(H, G, D, DV, T, window, keep):
    q, k, v = _attention_case(6, H, G, D, DV, T, window, keep)
    gate = torch.randn(T, H, generator=torch.Generator().manual_seed(7))
    scale, lam, diff, eps = 0.3, 0.45, 0.2, 1e-5
    ref = plain.difference_attention_heads(q.double(), k.double(), v.double(), scale, window or T + 1, keep, lam, diff, eps)
    ref = (ref * torch.sigmoid(gate.double())[:, :, None]).reshape(T, H * DV)
    for rows_form in (False, True):
        _close(_run_attention(q, k, v, window, keep, scale, lam, 1 - diff, eps, gate, rows_form), ref, 2e-5)
        for split in (1, 33, T - 2, T - 1):                 # rows on top of held ones, down to the last alone
            _close(_run_attention(q, k, v, window, keep, scale, lam, 1 - diff, eps, gate, rows_form, split=split), ref[split:], 2e-5)
    for shares in (2, 3, 16):                               # a row's keys cut over several blocks, more than it has tiles too
        _close(_run_attention(q, k, v, window, keep, scale, lam, 1 - diff, eps, gate, True, split=T - 9, shares=shares), ref[T - 9:], 2e-5)
    bf = _run_attention(q, k, v, window, keep, scale, lam, 1 - diff, eps, gate, False, dtype=torch.bfloat16)
    _close(bf, ref, 0.05)


@pytest.mark.parametrize("H, G, D, DV, T, window, keep", [
    (4, 2, 16, 16, 150, 9, 3), (3, 1, 32, 48, 200, 70, 0), (2, 2, 48, 80, 330, 36, 12), (2, 1, 64, 128, 260, 64, 32),
    (2, 1, 128, 64, 140, 0, 0), (1, 1, 16, 32, 66, 1, 1), (2, 2, 80, 112, 200, 130, 70)])
def test_two_maps_on_the_tensor_cores(H, G, D, DV, T, window, keep):
    """The bfloat16 tiles form on mma.sync against the plain statement on the same bfloat16 inputs: what is left is the
    output's own rounding."""
    q, k, v = (t.to(torch.bfloat16).float() for t in _attention_case(16, H, G, D, DV, T, window, keep))
    gate = torch.randn(T, H, generator=torch.Generator().manual_seed(17)).to(torch.bfloat16).float()
    scale, lam, diff, eps = D ** -0.5, 0.45, 0.2, 1e-5
    ref = plain.difference_attention_heads(q.double(), k.double(), v.double(), scale, window or T + 1, keep, lam, diff, eps)
    ref = (ref * torch.sigmoid(gate.double())[:, :, None]).reshape(T, H * DV)
    for split in (None, 1, 63, 64, T - 2):
        got = _run_attention(q, k, v, window, keep, scale, lam, 1 - diff, eps, gate, False, dtype=torch.bfloat16, split=split,
                             tensor_cores=True)
        _close(got, ref[split or 0:], 6e-3)
        err = (got.double().cpu() - ref[split or 0:]).abs() / ref.abs().max()
        assert float(err.mean()) < 1e-3                       # rounding of the output alone: a bfloat16 weight would show


@pytest.mark.parametrize("form", ["tiles", "rows", "mma"])
@pytest.mark.parametrize("window, keep, T", [(48, 24, 300), (9, 3, 70), (64, 0, 200), (33, 40, 129)])
def test_a_key_at_every_edge_decides_the_row(window, keep, T, form):
    """The last query's score with one key dwarfs the rest: just inside the window, just outside it, the last kept
    token, the first token that is not kept, a far key at a page border.  A mask that is one token off moves the result
    from one value row to another."""
    H, G, D, DV = 2, 1, 16, 16
    rows_form, mma = form == "rows", form == "mma"
    dtype, tol = (torch.bfloat16, 8e-3) if mma else (torch.float32, 2e-5)
    qi = T - 1
    spots = [qi - window + 1, qi - window, qi - window - 1, keep - 1, keep, 0, 63, 64, qi]
    for kj in spots:
        if not 0 <= kj <= qi:
            continue
        q, k, v = _attention_case(8, H, G, D, DV, T, window, keep, stand_out=(qi, kj))
        if mma:
            q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
        ref = plain.difference_attention_heads(q.double(), k.double(), v.double(), 1.0, window, keep, 0.1, 0.0, 1e-6)
        got = _run_attention(q, k, v, window, keep, 1.0, 0.1, 1.0, 1e-6, None, rows_form, split=T - 1 if rows_form else None,
                             dtype=dtype, tensor_cores=mma)
        _close(got[-1], ref[-1].reshape(-1), tol)
        # and the same query in a prompt's portion
        got = _run_attention(q, k, v, window, keep, 1.0, 0.1, 1.0, 1e-6, None, rows_form, split=max(0, T - 37), dtype=dtype,
                             tensor_cores=mma)
        _close(got[-1], ref[-1].reshape(-1), tol)
