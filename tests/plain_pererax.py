"""A plain, slow Pererax decoder in float64: whole sequences, no cache, one function per mechanism.

It shares no code with the package: it reads config.json and the safetensors file itself and
works on torch float64 tensors on the CPU.  `round_to` (a torch dtype or None) rounds where a
16-bit engine rounds: weights, the inputs of matrix products, cached keys and values.

Notation: x [T, E] is the residual stream; rms(v) = v / sqrt(mean(v^2) + eps).  A layer is

    x += ls1 * (rms(mixer(x)) * n1);   x += ls2 * (rms(ff(x)) * n2)

(the sublayers read x itself; the norm sits on their results).  The mixer is windowed attention whose
values are its unrotated keys, a gated delta rule with one decay per key channel, or the mean of a
sink attention and a matrix-memory recurrence, each RMS-normed first.  The feed-forward is a mixture
of clamped gated units with identity experts and one unit that every token runs through.  The output
is E_table (rms(x) * w_final).
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

F64 = torch.float64


# --------------------------------------------------------------------------- files
def read_safetensors(path):
    """name -> float64 (or int64) tensor."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    kinds = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        raw = bytearray(data[a:b])
        dt = meta["dtype"]
        if dt in kinds:
            t = torch.frombuffer(raw, dtype=kinds[dt]).to(F64) if raw else torch.zeros(0, dtype=F64)
        elif dt == "I32":
            t = torch.frombuffer(raw, dtype=torch.int32).to(torch.int64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = t.reshape(meta["shape"]).clone()
    return out


def load(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------- small functions
def rnd(t, round_to):
    return t if round_to is None else t.to(round_to).to(F64)


def rms(v, eps):
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def logsigmoid(z):
    return -softplus(-z)


def matmul(x, w, round_to):
    """x W^T with both operands rounded as a 16-bit engine rounds them."""
    return rnd(x, round_to) @ rnd(w, round_to).T


# --------------------------------------------------------------------------- positions and masks
def frequencies(base, dims):
    """f_i = base^(-2i/dims), i < dims/2."""
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def rotate_half(v, positions, base, dims):
    """v [T, heads, D]: element i < dims/2 of every head pairs with element i + dims/2 and the pair turns
    by position * f_i; elements from dims on pass."""
    out = v.clone()
    half = dims // 2
    ang = positions.to(F64)[:, None] * torch.tensor(frequencies(base, dims), dtype=F64)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def causal_mask(T, window=0):
    """[T, T] bool: query i sees key j <= i, and with a window only 0 <= i - j < window."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    return m & (i - j < window) if window else m


# --------------------------------------------------------------------------- attention
def whole_norm(p, w, eps):
    """RMS norm over a token's whole projection (all heads at once) with a plain weight."""
    return rms(p, eps) * w


def soft_cap(s, cap):
    return cap * torch.tanh(s / cap)


def masked_softmax(scores, mask, sink):
    """Softmax over the visible keys; with `sink` a key of score 0 and no value joins the denominator."""
    s = scores.masked_fill(~mask, -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink:
        m = torch.clamp(m, min=0.0)
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink:
        den = den + torch.exp(-m)
    return e / den


def attention(x, w, pre, m, eps, round_to=None, positions=None):
    """Grouped-query attention.  m: heads, kv_heads, dim, vdim, scale, rot {base, dims}, optional mask {size},
    optional softcap; `sink` and `value_is_key` in m say which of the two kinds it is."""
    T = x.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = positions if positions is not None else torch.arange(T)
    q = matmul(x, w[pre + "q"], round_to)
    k = matmul(x, w[pre + "k"], round_to)
    v = k.clone() if m.get("value_is_key") else matmul(x, w[pre + "v"], round_to)
    q = whole_norm(q, w[pre + "q.norm"], eps).reshape(T, H, D)
    k = whole_norm(k, w[pre + "k.norm"], eps).reshape(T, G, D)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, pos, rot["base"], rot["dims"])
        k = rotate_half(k, pos, rot["base"], rot["dims"])
    q, k, v = rnd(q, round_to), rnd(k, round_to), rnd(v.reshape(T, G, Dv), round_to)
    mask = causal_mask(T, (m.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, Dv, dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        if m.get("softcap"):
            s = soft_cap(s, m["softcap"])
        p = masked_softmax(s, mask, bool(m.get("sink")))
        out[:, h] = p @ v[:, g]
    return matmul(out.reshape(T, H * Dv), w[pre + "o"], round_to)


# --------------------------------------------------------------------------- matrix memory (mLSTM)
def capped(z, cap):
    return cap * torch.tanh(z / cap)


def matrix_memory_walk(q, k, v, ig, fg):
    """q, k [T, H, D] (q already scaled), v [T, H, Dv], ig / fg [T, H]: log input gate and log forget gate.
    With m_0 = 0, S_0 = 0, n_0 = 0:   m_t = max(f + m, i);  S_t = e^(f + m - m_t) S + e^(i - m_t) k v^T;
    n_t likewise with k;  o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6)."""
    T, H, D = q.shape
    Dv = v.shape[2]
    S = torch.zeros(H, D, Dv, dtype=F64)
    n = torch.zeros(H, D, dtype=F64)
    m = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a = torch.exp(fg[t] + m - m_new)
        b = torch.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out


def matrix_memory(x, w, pre, m, eps, round_to=None):
    T = x.shape[0]
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = matmul(x, w[pre + "q"], round_to).reshape(T, H, D) * D ** -0.5
    k = matmul(x, w[pre + "k"], round_to).reshape(T, H, D)
    v = matmul(x, w[pre + "v"], round_to).reshape(T, H, Dv)
    ig = capped(matmul(x, w[pre + "i"], round_to) + w[pre + "i.b"], cap)
    fg = logsigmoid(capped(matmul(x, w[pre + "f"], round_to) + w[pre + "f.b"], cap))
    o = rms(matrix_memory_walk(q, k, v, ig, fg), eps).reshape(T, H * Dv)
    o = o * w[pre + "norm"] * torch.sigmoid(matmul(x, w[pre + "g"], round_to))
    return matmul(o, w[pre + "o"], round_to)


def parallel_mixer(x, w, pre, m, eps, round_to=None):
    """Half the sum of the two branches, each RMS-normed over the width with its own weight first."""
    left = dict(m["left"], sink=True)
    a = rms(attention(x, w, pre + "left.", left, eps, round_to), eps) * w[pre + "left.out"]
    b = rms(matrix_memory(x, w, pre + "right.", m["right"], eps, round_to), eps) * w[pre + "right.out"]
    return 0.5 * (a + b)


# --------------------------------------------------------------------------- gated delta rule
def short_conv(u, taps_w):
    """u [T, C], taps_w [C, taps]: y[t, c] = sum_j taps_w[c, j] u[t - (taps - 1) + j, c], zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F64), u], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y = y + pad[j:j + T] * taps_w[:, j][None, :]
    return y


def unit(v):
    return v / torch.sqrt((v * v).sum(dim=-1, keepdim=True) + 1e-6)


def delta_walk(q, k, v, beta, g):
    """q, k [T, H, D], v [T, H, Dv], beta [T, H], g [T, H, D] (decay per key channel), S_0 = 0:
    S <- g * S (rows);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, H, D = q.shape
    Dv = v.shape[2]
    S = torch.zeros(H, D, Dv, dtype=F64)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for t in range(T):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def channel_delta(x, w, pre, m, eps, round_to=None):
    T = x.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rep = H // G
    q = silu(short_conv(matmul(x, w[pre + "q"], round_to), w[pre + "q.conv"])).reshape(T, G, D)
    k = silu(short_conv(matmul(x, w[pre + "k"], round_to), w[pre + "k.conv"])).reshape(T, G, D)
    v = silu(short_conv(matmul(x, w[pre + "v"], round_to), w[pre + "v.conv"])).reshape(T, H, Dv)
    q = (unit(q) * D ** -0.5).repeat_interleave(rep, dim=1)
    k = unit(k).repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(matmul(x, w[pre + "b"], round_to))
    low = matmul(matmul(x, w[pre + "a1"], round_to), w[pre + "a2"], round_to) + w[pre + "dt_bias"]
    g = torch.exp(-torch.exp(w[pre + "A_log"])[None, :, None] * softplus(low).reshape(T, H, D))
    o = rms(delta_walk(q, k, v, beta, g), eps) * w[pre + "norm"]
    gate = torch.sigmoid(matmul(matmul(x, w[pre + "g1"], round_to), w[pre + "g2"], round_to)).reshape(T, H, Dv)
    return matmul((o * gate).reshape(T, H * Dv), w[pre + "o"], round_to)


# --------------------------------------------------------------------------- feed-forward
def clamped_unit(x, w, pre, limit, round_to=None):
    """down(g sigmoid(1.702 g) (u + 1)) with g = min(gate x, limit), u = clamp(up x, -limit, limit)."""
    g = torch.clamp(matmul(x, w[pre + "gate"], round_to), max=limit)
    u = torch.clamp(matmul(x, w[pre + "up"], round_to), min=-limit, max=limit)
    return matmul(g * torch.sigmoid(1.702 * g) * (u + 1.0), w[pre + "down"], round_to)


def route(x, w, pre, r, round_to=None, margins=None):
    """(chosen [T, top] indices, weights [T, top], scores [T, n]): softmax scores over experts + identity
    outputs; the choice adds the correction vector, the weights do not and are scaled, not renormalised.
    `margins` (a list) receives, per token, by how much the last chosen output beats the first one left out,
    in units of the spread of the token's scores (infinite when every output is chosen)."""
    z = matmul(x, w[pre + "router"], round_to)
    s = torch.softmax(z, dim=-1)
    pick = s + w[pre + "correction"]
    # a tie goes to the lower index: stable sort, descending
    order = torch.sort(pick, dim=-1, descending=True, stable=True)
    idx = order.indices[:, :r["top"]]
    if margins is not None:
        if pick.shape[1] > r["top"]:
            margins.append((order.values[:, r["top"] - 1] - order.values[:, r["top"]]) / s.std(dim=-1).clamp_min(1e-30))
        else:
            margins.append(torch.full((x.shape[0],), math.inf, dtype=F64))
    return idx, torch.gather(s, 1, idx) * r.get("scale", 1.0), s


def mixture(x, w, pre, mlp, round_to=None, margins=None):
    r = mlp["router"]
    n_real, n_id = r["experts"], r.get("identity", 0)
    idx, wt, _ = route(x, w, pre, r, round_to, margins)
    y = torch.zeros_like(x)
    xr = rnd(x, round_to)
    for e in range(n_real + n_id):
        hit = idx == e
        rows = hit.any(dim=-1)
        if not rows.any():
            continue
        we = (wt * hit).sum(dim=-1)[rows]
        res = clamped_unit(x[rows], w, f"{pre}e{e}.", mlp["expert"]["limit"], round_to) if e < n_real else xr[rows]
        y[rows] = y[rows] + we[:, None] * res
    if mlp.get("shared"):
        y = y + clamped_unit(x, w, pre + "shared.", mlp["shared"]["limit"], round_to)
    return y


# --------------------------------------------------------------------------- the model
def weights_owner(layers, i):
    while layers[i].get("weights_of") is not None:
        i = layers[i]["weights_of"]
    return i


def mixer(kind, x, w, pre, m, eps, round_to=None):
    if kind == "attention":
        return attention(x, w, pre, dict(m, value_is_key=True), eps, round_to)
    if kind == "parallel":
        return parallel_mixer(x, w, pre, m, eps, round_to)
    if kind == "channel_delta":
        return channel_delta(x, w, pre, m, eps, round_to)
    raise ValueError(kind)


def forward(cfg, w, tokens, round_to=None, trace=None, margins=None):
    """Logits [T, vocab] of one sequence; `trace` (a list) receives x after every layer, `margins` (a list) every
    router's margins per token (see `route`)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)].clone()
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{weights_owner(cfg['layers'], i)}."
        y = mixer(layer["type"], x, w, p + "mix.", layer["mixer"], eps, round_to)
        x = x + w[p + "ls1"] * (rms(y, eps) * w[p + "norm1"])
        if layer.get("mlp"):
            y = mixture(x, w, p + "mlp.", layer["mlp"], round_to, margins)
            x = x + w[p + "ls2"] * (rms(y, eps) * w[p + "norm2"])
        if trace is not None:
            trace.append(x.clone())
    return matmul(rms(x, eps) * w["final.norm"], w["embed"], round_to)
