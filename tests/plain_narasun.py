"""Plain, slow statement of the Narasun decoder: one function per mechanism, token by token where a
mechanism is recurrent, float64 unless told otherwise.  It shares no code with the library: tensors come
in as a dict {name: torch tensor}, the configuration as the dict of config.json.

Notation: x residual stream [T, W]; h = norm(x); a sequence is processed from its position 0, so
functions take whole sequences and return whole sequences.  `rd` is the identity, or a rounding to
bfloat16 applied where a bfloat16 engine stores activations (norm outputs, projections, activations,
the mixers' outputs before the last projection): with it the result shows how much noise the storage
format alone causes on an input, which is the yardstick for the bfloat16 engine.
"""
import math

import torch


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the distance from one."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def ident(x):
    return x


def to_bf16(x):
    return x.to(torch.bfloat16).to(x.dtype)


def swiglu(h, wg, wu, wd, rd=ident):
    return rd(silu(h @ wg.T) * (h @ wu.T)) @ wd.T


def dense_ff(t, p, h, rd=ident):
    return swiglu(h, t[p + "gate"], t[p + "up"], t[p + "down"], rd)


def moe_ff(t, p, h, n_experts, top, rd=ident, choice=None):
    """Sigmoid router; the `top` best experts; each gets score * h as its input; outputs added.
    choice ([tokens, top] expert ids) replaces the router's decision (not its scores): a comparison with an
    engine in a format whose rounding may turn a close call the other way then rests on the arithmetic alone."""
    z = h @ t[p + "router"].T
    s = torch.sigmoid(z)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        order = sorted(range(n_experts), key=lambda e: (-float(s[i, e]), e))[:top]
        if choice is not None:
            order = [int(e) for e in choice[i]]
        for e in order:
            q = f"{p}e{e}."
            out[i] += swiglu(rd(s[i, e] * h[i]), t[q + "gate"], t[q + "up"], t[q + "down"], rd)
    return out


def sink_attention_heads(q, k, v, sink, scale, coef, every, first=0):
    """q [T, H, D] at positions first .. first + T - 1, k [S, G, D], v [S, G, DV] at positions 0 .. S - 1
    (S >= first + T).  Causal, grouped heads, no rotation; a per-head sink logit joins the denominator;
    queries are multiplied by 1 + coef ln(floor((p + 1) / every) + 1).  Returns [T, H, DV]."""
    T, H, _ = q.shape
    S, G, DV = v.shape
    pos = torch.arange(first, first + T)
    temp = torch.ones(T, dtype=q.dtype)
    if every:
        temp = 1.0 + coef * torch.log(torch.div(pos + 1, every, rounding_mode="floor").to(q.dtype) + 1.0)
    hidden = torch.arange(S)[None, :] > pos[:, None]
    out = torch.zeros(T, H, DV, dtype=q.dtype)
    for a in range(H):
        g = a // (H // G)
        sc = ((q[:, a] * temp[:, None]) @ k[:, g].T) * scale
        sc = sc.masked_fill(hidden, float("-inf"))
        m = torch.maximum(sc.max(-1).values, sink[a].expand(T))
        e = torch.exp(sc - m[:, None])
        den = e.sum(-1) + torch.exp(sink[a] - m)
        out[:, a] = (e @ v[:, g]) / den[:, None]
    return out


def sink_attention(t, p, h, c, rd=ident):
    T = h.shape[0]
    H, G, D, DV = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = rd(h @ t[p + "q"].T).view(T, H, D)
    k = rd(h @ t[p + "k"].T).view(T, G, D)
    v = rd(h @ t[p + "v"].T).view(T, G, DV)
    qt = c.get("q_temp") or {"coef": 0.0, "every": 0}
    o = sink_attention_heads(q, k, v, t[p + "sink"], c["scale"], qt["coef"], qt["every"])
    return rd(o).reshape(T, H * DV) @ t[p + "o"].T


def decay_mix(t, p, h, c, eps, rd=ident):
    """Time mixing with a per-channel, per-token decay and a bonus for the present token."""
    T, W = h.shape
    H, D = c["heads"], c["dim"]
    prev = torch.cat([torch.zeros(1, W, dtype=h.dtype), h[:-1]], 0)
    mix = {s: rd(h + (prev - h) * t[p + "mu." + s]) for s in "rkvgw"}
    r = rd(mix["r"] @ t[p + "r"].T).view(T, H, D)
    k = rd(mix["k"] @ t[p + "k"].T).view(T, H, D)
    v = rd(mix["v"] @ t[p + "v"].T).view(T, H, D)
    gate = silu(rd(mix["g"] @ t[p + "g"].T))
    w = torch.exp(-torch.exp(torch.tanh(mix["w"] @ t[p + "w1"].T) @ t[p + "w2"].T + t[p + "w0"])).view(T, H, D)
    u = t[p + "u"]
    S = torch.zeros(H, D, D, dtype=h.dtype)
    o = torch.zeros(T, H, D, dtype=h.dtype)
    for i in range(T):
        kv = k[i][:, :, None] * v[i][:, None, :]
        o[i] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[i])
        S = w[i][:, :, None] * S + kv
    o = rms_unit(o, eps).reshape(T, H * D) * t[p + "norm"] * gate
    return rd(o) @ t[p + "o"].T


def matrix_memory(t, p, h, c, eps, rd=ident):
    """mLSTM: exponential input gate, sigmoid forget gate in the log domain with a running maximum that
    starts at zero, a normaliser vector beside the matrix."""
    T = h.shape[0]
    H, D, DV, cap = c["heads"], c["dim"], c["vdim"], c["gate_cap"]
    q = rd(h @ t[p + "q"].T).view(T, H, D) * D ** -0.5
    k = rd(h @ t[p + "k"].T).view(T, H, D)
    v = rd(h @ t[p + "v"].T).view(T, H, DV)
    ig = cap * torch.tanh((h @ t[p + "i"].T + t[p + "i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ t[p + "f"].T + t[p + "f.b"]) / cap))
    S = torch.zeros(H, D, DV, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    m = torch.zeros(H, dtype=h.dtype)
    o = torch.zeros(T, H, DV, dtype=h.dtype)
    for i in range(T):
        m_new = torch.maximum(fg[i] + m, ig[i])
        a, b = torch.exp(fg[i] + m - m_new), torch.exp(ig[i] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * (k[i][:, :, None] * v[i][:, None, :])
        n = a[:, None] * n + b[:, None] * k[i]
        m = m_new
        num = torch.einsum("hkv,hk->hv", S, q[i])
        den = torch.maximum((n * q[i]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        o[i] = num / den[:, None]
    o = rms_unit(o, eps).reshape(T, H * DV) * t[p + "norm"] * torch.sigmoid(rd(h @ t[p + "g"].T))
    return rd(o) @ t[p + "o"].T


def base_kind(kind):
    """'mlstm_2' and 'mlstm' name the same mixer."""
    head, _, tail = kind.rpartition("_")
    return head if head and tail.isdigit() else kind


def mixer(t, l, h, layer, eps, rd=ident):
    kind, c, p = base_kind(layer["type"]), layer["mixer"], f"l{l}.mix."
    if kind == "parallel":
        return (c["left_scale"] * sink_attention(t, p + "left.", h, c["left"], rd)
                + c["right_scale"] * decay_mix(t, p + "right.", h, c["right"], eps, rd))
    if kind == "mlstm":
        return matrix_memory(t, p, h, c, eps, rd)
    raise ValueError(kind)


def feed_forward(t, l, h, mlp, rd=ident, choice=None):
    if mlp is None:
        return torch.zeros_like(h)
    if mlp["kind"] == "dense":
        return dense_ff(t, f"l{l}.mlp.", h, rd)
    return moe_ff(t, f"l{l}.mlp.", h, mlp["router"]["experts"], mlp["router"]["top"], rd, choice)


def layer_order(cfg):
    """[(layer, pass number or None when the pass does not begin here)]"""
    L, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(l, None) for l in range(L)]
    out = [(l, None) for l in range(loop["start"])]
    for t_ in range(loop["times"]):
        for l in range(loop["start"], loop["stop"]):
            out.append((l, t_ if l == loop["start"] else None))
    out += [(l, None) for l in range(loop["stop"], L)]
    return out


def forward(cfg, t, tokens, dtype=torch.float64, streams=None, bf16=False, choices=None):
    """Logits [T, vocab] of one sequence from its first token; `streams` (a list) receives the residual
    stream after every layer run.  bf16: round where a bfloat16 engine stores activations.  choices: per run
    of a routed feed-forward, in the order of the runs, the experts to use ([tokens, top]; see moe_ff)."""
    rd = to_bf16 if bf16 else ident
    routed = 0
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in t.items()}
    eps = cfg["norm"]["eps"]
    x = t["embed"][torch.as_tensor(tokens)]
    x0 = x.clone()
    for l, begins in layer_order(cfg):
        if begins is not None:
            x = rd(torch.cat([x, x0], -1)) @ t["loop.in"].T + t["loop.step"][begins]
        layer = cfg["layers"][l]
        h = rd(offset_norm(x, t[f"l{l}.norm1"], eps))
        choice = None
        if choices is not None and (layer.get("mlp") or {}).get("kind") == "moe":
            choice, routed = choices[routed], routed + 1
        x = x + (mixer(t, l, h, layer, eps, rd) + feed_forward(t, l, h, layer.get("mlp"), rd, choice))
        if streams is not None:
            streams.append(x.clone())
    return rd(offset_norm(x, t["final.norm"], eps)) @ t["head"].T


def greedy(cfg, t, prompt, n_new):
    """n_new tokens, each the first of the largest logits after everything before it."""
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(torch.argmax(forward(cfg, t, tokens)[-1])))
    return tokens[len(prompt):]
