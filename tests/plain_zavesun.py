"""A plain, slow Zavesun decoder in float64: whole sequences, no cache, one function per mechanism.

It shares no code with the package: it reads config.json and the safetensors file itself and
works on torch float64 tensors on the CPU.  `round_to` (a torch dtype or None) rounds where a
16-bit engine rounds: weights, the inputs of matrix products, cached keys and values.

Notation: the model carries S copies X[0..S-1] of the residual stream, each [T, E], all equal to
the embedded tokens at the start.  A sublayer f (mixer, then feed-forward) with its three small
tensors a [S] (read), M [S, S] (carry, indexed [from, to]) and b [S] (write) does

    u = sum_s a[s] X[s];   y = f(rms(u) * w);   X'[t] = sum_s M[s, t] X[s] + b[t] * y      (all t at once)

with rms(v) = v / sqrt(mean(v^2) + eps).  The output is softcap(E_table rms(sum_s X[s]) * w_final).
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def matmul(x, w, round_to):
    """x W^T with both operands rounded as a 16-bit engine rounds them."""
    return rnd(x, round_to) @ rnd(w, round_to).T


# --------------------------------------------------------------------------- positions
def linear_frequencies(base, dims, factor=1.0):
    """f_i = base^(-2i/dims) / factor, i < dims/2."""
    return [base ** (-2.0 * i / dims) / factor for i in range(dims // 2)]


def rotate_interleaved(v, positions, freqs, dims):
    """v [T, heads, D]: elements (2i, 2i+1), i < dims/2, of every head turn by position * freqs[i]."""
    out = v.clone()
    ang = positions.to(F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    steps = torch.div(positions + 1, every, rounding_mode="floor").to(F64)
    return 1.0 + coef * torch.log(steps + 1.0)


def head_slopes(heads):
    """2^(-8 (h + 1) / heads) for h = 0 .. heads-1."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F64)


# --------------------------------------------------------------------------- masks
def window_mask(T, size):
    """[T, T] bool: query i sees key j when 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def chunk_mask(T, size):
    """[T, T] bool: query i sees key j <= i of its own chunk of `size` positions (chunks start at position 0)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))


def softmax_attention(q, k, v, scale, mask, bias=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; head h reads key/value head h // (H/G).  bias [H, T, T]
    is taken off the scaled scores.  Returns [T, H * Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = []
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        if bias is not None:
            s = s - bias[h]
        s = s.masked_fill(~mask, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, h // rep])
    return torch.cat(out, dim=-1)


def mix_values(v, v_first, lam):
    """(1 - lam) v + lam v_first."""
    return (1.0 - lam) * v + lam * v_first


# --------------------------------------------------------------------------- mixers
def attention_windowed(h, W, p, m, carry, is_first, round_to):
    """The `attention` mixer: no rotation; queries scaled by a temperature of their position; a
    distance bias slope_h * (i - j); a sliding window; values mixed with the first mixing layer's."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = matmul(h, W[p + "q"], round_to).view(T, H, D)
    k = matmul(h, W[p + "k"], round_to).view(T, G, D)
    v = matmul(h, W[p + "v"], round_to).view(T, G, Dv)
    if m.get("q_temp"):
        q = q * query_temperature(pos, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]))[:, None, None]
    v = _value_mix(v, W, p, m, carry, is_first)
    dist = (pos[:, None] - pos[None, :]).to(F64)
    bias = head_slopes(H)[:, None, None] * dist[None]
    mask = window_mask(T, int(m["mask"]["size"])) if m.get("mask") else window_mask(T, T + 1)
    y = softmax_attention(rnd(q, round_to), rnd(k, round_to), rnd(v, round_to), float(m["scale"]), mask, bias)
    return matmul(y, W[p + "o"], round_to)


def attention_chunked(h, W, p, m, eps, carry, is_first, round_to):
    """The `attention_2` mixer: biased projections, a weighted RMS norm of every query and key head,
    a partial interleaved rotation with divided frequencies, chunked visibility, mixed values."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (matmul(h, W[p + "q"], round_to) + W[p + "q.b"]).view(T, H, D)
    k = (matmul(h, W[p + "k"], round_to) + W[p + "k.b"]).view(T, G, D)
    v = (matmul(h, W[p + "v"], round_to) + W[p + "v.b"]).view(T, G, Dv)
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    rot = m.get("rot")
    if rot:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        f = linear_frequencies(float(rot["base"]), int(rot["dims"]), factor)
        q = rotate_interleaved(q, pos, f, int(rot["dims"]))
        k = rotate_interleaved(k, pos, f, int(rot["dims"]))
    v = _value_mix(v, W, p, m, carry, is_first)
    mask = chunk_mask(T, int(m["mask"]["size"])) if m.get("mask") else window_mask(T, T + 1)
    y = softmax_attention(rnd(q, round_to), rnd(k, round_to), rnd(v, round_to), float(m["scale"]), mask)
    return matmul(y, W[p + "o"], round_to)


def _value_mix(v, W, p, m, carry, is_first):
    if not m.get("v_mix"):
        return v
    if is_first:
        carry["v_first"] = v
        return v
    return mix_values(v, carry["v_first"].view_as(v), W[p + "vmix"])


# --------------------------------------------------------------------------- feed-forwards
def dense_ff(h, W, p, round_to):
    """down(gelu_tanh(gate h) * (up h))."""
    a = gelu_tanh(matmul(h, W[p + "gate"], round_to)) * matmul(h, W[p + "up"], round_to)
    return matmul(a, W[p + "down"], round_to)


def router_choice(h, w_router, top, round_to):
    """(indices [T, top], weights [T, top]): the `top` largest sigmoid scores, as they are."""
    s = torch.sigmoid(matmul(h, w_router, round_to))
    w, idx = torch.topk(s, top, dim=-1)
    return idx, w


def router_margin(h, w_router, top, round_to):
    """[T]: how far the last chosen logit lies above the best one left out, in standard deviations of all the
    logits (inf when every expert is chosen)."""
    z = matmul(h, w_router, round_to)
    s = z.sort(dim=-1, descending=True).values
    if s.shape[1] <= top:
        return torch.full((h.shape[0],), float("inf"), dtype=F64)
    return (s[:, top - 1] - s[:, top]) / z.std()


def routed_ff(h, W, p, mlp, round_to, margins=None):
    """sum over a token's chosen experts of expert(weight * h); expert = down(silu(gate z) * (up z)).
    margins, a list, receives this layer's `router_margin`."""
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    idx, w = router_choice(h, W[p + "router"], top, round_to)
    if margins is not None:
        margins.append(router_margin(h, W[p + "router"], top, round_to))
    y = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for e in range(n):
        for j in range(top):
            rows = (idx[:, j] == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            z = h[rows] * w[rows, j:j + 1]
            q = f"{p}e{e}."
            a = silu(matmul(z, W[q + "gate"], round_to)) * matmul(z, W[q + "up"], round_to)
            y[rows] += matmul(a, W[q + "down"], round_to)
    return y


# --------------------------------------------------------------------------- streams
def streams_read(X, a):
    """u = sum_s a[s] X[s];  X [S, T, E]."""
    return torch.einsum("s,ste->te", a, X)


def streams_write(X, M, b, y):
    """X'[t] = sum_s M[s, t] X[s] + b[t] y."""
    return torch.einsum("st,sne->tne", M, X) + b[:, None, None] * y[None]


# --------------------------------------------------------------------------- the model
def forward(cfg, W, tokens, round_to=None, layers_out=None, margins=None):
    """Logits [T, vocab] (float64) of one sequence from position 0.  layers_out, a list, receives the
    sum of the streams [T, E] after every layer; margins, a list, every routed layer's `router_margin`."""
    eps = float(cfg["norm"]["eps"])
    S = int(cfg.get("streams", 1))
    W = {k: (rnd(v, round_to) if v.dim() >= 2 else v) for k, v in W.items()}
    tok = torch.as_tensor(tokens, dtype=torch.int64)
    x0 = W["embed"][tok]
    X = x0[None].repeat(S, 1, 1)
    carry = {}
    first_mix = next((i for i, L in enumerate(cfg["layers"]) if L["mixer"].get("v_mix")), None)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]

        def mixer(h):
            if L["type"] == "attention":
                return attention_windowed(h, W, p + "mix.", m, carry, i == first_mix, round_to)
            if L["type"] == "attention_2":
                return attention_chunked(h, W, p + "mix.", m, eps, carry, i == first_mix, round_to)
            raise ValueError(L["type"])

        def ff(h):
            if L["mlp"]["kind"] == "dense":
                return dense_ff(h, W, p + "mlp.", round_to)
            return routed_ff(h, W, p + "mlp.", L["mlp"], round_to, margins)

        subs = [(mixer, "1")] + ([(ff, "2")] if L.get("mlp") is not None else [])
        for f, q in subs:
            if S > 1 or (p + "hc" + q + ".in") in W:
                u = streams_read(X, W[p + "hc" + q + ".in"])
                y = f(rms(u, eps) * W[p + "norm" + q])
                X = streams_write(X, W[p + "hc" + q + ".mix"], W[p + "hc" + q + ".out"], y)
            else:
                X = X + f(rms(X[0], eps) * W[p + "norm" + q])[None]
        if layers_out is not None:
            layers_out.append(X.sum(dim=0))
    x = X.sum(dim=0)
    logits = matmul(rms(x, eps) * W["final.norm"], W["embed"], round_to)
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits
