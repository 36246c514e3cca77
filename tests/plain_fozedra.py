"""Plain, slow statement of the Fozedra decoder: one function per mechanism, float64 unless told otherwise.
It shares no code with the library: tensors come in as a dict {name: torch tensor}, the configuration as
the dict of config.json.

Notation: x residual stream [T, W]; a sequence is processed from its position 0, so functions take whole
sequences and return whole sequences.  `rd` is the identity, or a rounding to bfloat16 applied where a
bfloat16 engine stores activations (norm outputs, projections and their activations, the mixers' outputs
before the last projection): with it the result shows how much noise the storage format alone causes,
which is the yardstick for the bfloat16 engine.

The layer:  x <- x + m * mixer(dyt(x; norm1)),  then (if the layer has one)  x <- x + m * ff(dyt(x; norm2)).
"""
import math

import torch


def ident(x):
    return x


def to_bf16(x):
    return x.to(torch.bfloat16).to(x.dtype)


def silu(z):
    return z * torch.sigmoid(z)


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyt(x, alpha, w, b):
    """Dynamic tanh in place of a norm: no statistics of the row are taken."""
    return torch.tanh(alpha * x) * w + b


def relu2_ff(h, w_up, w_down, rd=ident):
    z = torch.relu(rd(h @ w_up.T))
    return rd(z * z) @ w_down.T


def causal_taps(u, w):
    """u [T, C], w [C, K]: y_t = sum_j w[:, j] * u_(t - K + 1 + j), zeros before the sequence's start."""
    T, C = u.shape
    K = w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + padded[j:j + T] * w[:, j]
    return y


def yarn_rates(dims, base, factor, original, fast, slow):
    """Per-pair angular rates [dims / 2] and the factor on cosine and sine."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(fast)), 0)
    hi = min(math.ceil(turn_dim(slow)), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_front(x, first, dims, rates, mag):
    """x [T, n, D] at positions first ..: the leading `dims` channels of every vector are turned, channel i
    against channel i + dims/2; the others pass."""
    T = x.shape[0]
    half = dims // 2
    pos = torch.arange(first, first + T, dtype=x.dtype)
    ang = pos[:, None] * torch.tensor(rates, dtype=x.dtype)[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def visible(T, size, keep_first):
    """[T, T] bool: query i sees key j."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def difference_attention_heads(q, k, v, scale, size, keep_first, lam, diff, eps):
    """q [T, H, 2, D], k [T, G, 2, D], v [T, G, DV], all from position 0.  Two softmax maps over the same
    values; o = a1 - lam * a2, brought to unit root mean square per head, times (1 - diff).  Returns [T, H, DV]."""
    T, H = q.shape[:2]
    G, DV = v.shape[1:]
    see = visible(T, size, keep_first)
    out = torch.zeros(T, H, DV, dtype=q.dtype)
    for a in range(H):
        g = a // (H // G)
        maps = []
        for m in range(2):
            sc = (q[:, a, m] @ k[:, g, m].T) * scale
            sc = sc.masked_fill(~see, float("-inf"))
            maps.append(torch.softmax(sc, -1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, a] = rms_unit(o, eps) * (1.0 - diff)
    return out


def attention_kv(t, p, mx, h, rd=ident):
    """The keys (after taps and rotation) [T, G, 2, D] and values (after taps) [T, G, DV] of a layer that has
    projections of its own."""
    G, D, DV = mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    k = causal_taps(rd(h @ t[p + "k"].T + t[p + "k.b"]), t[p + "k.conv"])
    v = causal_taps(rd(h @ t[p + "v"].T + t[p + "v.b"]), t[p + "v.conv"])
    rot = mx["rot"]
    sc = rot["scaling"]
    rates, mag = yarn_rates(rot["dims"], rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
    k = rotate_front(k.view(T, G * 2, D), 0, rot["dims"], rates, mag).view(T, G, 2, D)
    return rd(k), rd(v).view(T, G, DV)


def attention_mixer(t, p, mx, h, eps, kv=None, rd=ident):
    """kv: another layer's (keys, values) for a layer that has none of its own.  Returns (output, (keys, values))."""
    H, D, DV = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    if kv is None:
        kv = attention_kv(t, p, mx, h, rd)
    k, v = kv
    q = causal_taps(rd(h @ t[p + "q"].T + t[p + "q.b"]), t[p + "q.conv"])
    rot = mx["rot"]
    sc = rot["scaling"]
    rates, mag = yarn_rates(rot["dims"], rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
    q = rd(rotate_front(q.view(T, H * 2, D), 0, rot["dims"], rates, mag)).view(T, H, 2, D)
    f32 = lambda name: t[p + name].to(torch.float32)
    lam = float(torch.exp((f32("lq1") * f32("lk1")).sum()) - torch.exp((f32("lq2") * f32("lk2")).sum())) + mx["diff"]
    o = difference_attention_heads(q, k, v, mx["scale"], mx["mask"]["size"], mx["mask"]["keep_first"], lam, mx["diff"], eps)
    gate = torch.sigmoid(h @ t[p + "g"].T)                       # [T, H]
    o = rd(o * gate[:, :, None]).reshape(T, H * DV)
    return o @ t[p + "o"].T, kv


def lightning_heads(q, k, v, decay):
    """q, k [T, H, D], v [T, H, DV], decay [H]: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token."""
    T, H, D = q.shape
    DV = v.shape[2]
    S = torch.zeros(H, D, DV, dtype=q.dtype)
    out = torch.zeros(T, H, DV, dtype=q.dtype)
    for i in range(T):
        S = S * decay[:, None, None] + k[i][:, :, None] * v[i][:, None, :]
        out[i] = torch.einsum("hdv,hd->hv", S, q[i])
    return out


def lightning_mixer(t, p, mx, h, eps, rd=ident):
    H, D, DV = mx["heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = rd(silu(rd(h @ t[p + "q"].T))).view(T, H, D)
    k = rd(silu(rd(h @ t[p + "k"].T))).view(T, H, D)
    v = rd(silu(rd(h @ t[p + "v"].T))).view(T, H, DV)
    o = lightning_heads(q, k, v, torch.tensor(mx["decay"], dtype=h.dtype)).reshape(T, H * DV)
    o = rms_unit(o, eps) * t[p + "norm"] * torch.sigmoid(h @ t[p + "g"].T)
    return rd(o) @ t[p + "o"].T


def forward(cfg, tensors, tokens, dtype=torch.float64, rd=ident, layers_out=None):
    """Logits [T, vocab] for one sequence from position 0.  layers_out: a list that receives the residual
    stream after every layer."""
    t = {n: w.to(dtype) for n, w in tensors.items()}
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    norm = lambda name, x: rd(dyt(x, t[name + ".alpha"], t[name], t[name + ".b"]))
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.mix.", layer["mixer"]
        h = norm(f"l{i}.norm1", x)
        if layer["type"] == "lightning":
            y = lightning_mixer(t, p, mx, h, eps, rd)
        else:
            y, kept[i] = attention_mixer(t, p, mx, h, eps, kept[mx["kv_from"]] if mx.get("kv_from") is not None else None, rd)
        x = x + m * y
        if layer.get("mlp") is not None:
            x = x + m * relu2_ff(norm(f"l{i}.norm2", x), t[f"l{i}.mlp.up"], t[f"l{i}.mlp.down"], rd)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm("final.norm", x) @ t["embed"].T
