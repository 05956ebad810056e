"""A plain, slow Rizovik: one function per mechanism, whole sequences at once, no cache.

Written from the design's equations with torch on the CPU; it shares no code with the engine and
is the oracle of the tests.  Notation: x is the residual stream [T, W]; matrices are stored
[out, in] and applied as ``h @ W.T``; positions are 0 .. T-1; rms(y) = y / sqrt(mean(y^2) + eps).

    embedding        x = E[token]
    layer            x = x + m n1(mixer(x));  x = x + m n2(ff(x))     (the sublayers read x itself; n(y) = rms(y) * w)
                     a layer with weights_of j runs layer j's tensors over a cache or state of its own
    pooled attention q, k RMS-normalised as whole projections (weights as long as the projection), the first
                     ``rot.dims`` elements of each head rotated (pairs i, i + dims/2), every head's value divided
                     by its root mean square; query i sees the keys j with 0 <= i - j < size and, for every block
                     of ``pool`` positions that ends at or before i - size, the mean of the block's keys and the
                     mean of its values; one softmax over both; heads times sigmoid(W_g x); W_o
    kept-first attention
                     q, k RMS-normalised per head with one weight [dim] for all heads, rotated with frequencies
                     divided by ``rot.scaling.factor``; query i sees j <= i with i - j < size or j < keep_first;
                     softmax; the heads' weights are mixed, w'_h = sum_g talk[h, g] w_g, and head h applies w'_h to
                     the values of its own KV head; W_o
    delta            q, k, v through a causal convolution per channel (zeros before the start) and silu; q, k made
                     unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times dim^(-1/2);
                     beta = sigmoid(W_b x); g = exp(-exp(A_log) softplus(W_a x + dt_bias)) per head;
                     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
                     per head rms(o) * w, times silu(W_g x); W_o
    routed ff        z = W_r x + b; the ``top`` largest z; weights softmax over the chosen z;
                     experts W_down (silu(W_gate x) * W_up x)
    output           logits = E n_final(x)
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# ---- files ---------------------------------------------------------------------------------------
def read_safetensors(path) -> dict[str, torch.Tensor]:
    data = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = bytearray(data[8 + n + a: 8 + n + b])
        out[name] = torch.frombuffer(buf, dtype=kinds[info["dtype"]]).reshape(info["shape"]).clone()
    return out


def load_folder(folder, dtype=torch.float64):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: (v.to(dtype) if v.is_floating_point() else v)
         for k, v in read_safetensors(folder / "model.safetensors").items()}
    return cfg, w


# ---- small functions -------------------------------------------------------------------------------
def unit_rms(y, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def rotate_half_split(t, positions, dims, base, factor=1.0):
    """t [T, n, d]: element i of the first ``dims`` turns together with element i + dims/2 by the angle
    position * base^(-2i/dims) / factor."""
    half = dims // 2
    i = torch.arange(half, dtype=t.dtype)
    f = base ** (-2.0 * i / dims) / factor
    a = positions.to(t.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = t[..., :half], t[..., half:dims]
    return torch.cat((u * c - v * s, v * c + u * s, t[..., dims:]), -1)


# ---- pooled-window attention -------------------------------------------------------------------------
def pooled_window_softmax(q, k, v, scale, size, pool, qpos=None):
    """q [R, H, d] at the positions ``qpos`` (default 0 .. R-1), k [L, G, d], v [L, G, dv] as cached.  Query i sees the
    positions j with 0 <= i - j < size and the mean key and value of every block of ``pool`` positions that ends at or
    before i - size; one softmax over both.  Returns [R, H, dv]."""
    R, H, _ = q.shape
    G = k.shape[1]
    qpos = list(range(R)) if qpos is None else [int(p) for p in qpos]
    nb = k.shape[0] // pool
    kb = k[:nb * pool].reshape(nb, pool, G, k.shape[-1]).mean(1)
    vb = v[:nb * pool].reshape(nb, pool, G, v.shape[-1]).mean(1)
    out = torch.zeros(R, H, v.shape[-1], dtype=q.dtype)
    for r, i in enumerate(qpos):
        lo = max(0, i - size + 1)
        seen = max(0, (i - size + 1) // pool)          # blocks whose last position is <= i - size
        for hd in range(H):
            g = hd // (H // G)
            keys = torch.cat((kb[:seen, g], k[lo:i + 1, g]), 0)
            vals = torch.cat((vb[:seen, g], v[lo:i + 1, g]), 0)
            out[r, hd] = torch.softmax(keys @ q[r, hd] * scale, 0) @ vals
    return out


def pooled_window_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (unit_rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]).view(T, H, d)
    k = (unit_rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]).view(T, G, d)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    if rot["dims"]:
        q = rotate_half_split(q, pos, rot["dims"], rot["base"])
        k = rotate_half_split(k, pos, rot["dims"], rot["base"])
    v = unit_rms((h @ w[p + "v"].T).view(T, G, dv), eps)
    out = pooled_window_softmax(q, k, v, m["scale"], m["mask"]["size"], m["mask"]["pool"])
    out = out.reshape(T, H * dv) * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---- attention with kept first tokens and mixed heads ------------------------------------------------
def kept_first_mixed(q, k, v, talk, scale, size, keep, qpos=None):
    """q [R, H, d] at ``qpos``, k [L, G, d], v [L, G, dv].  Query i sees j <= i with i - j < size or j < keep; after the
    softmax head h's weights become sum_g talk[h, g] w_g, applied to the values of h's own KV head.  [R, H, dv]."""
    R, H, _ = q.shape
    L, G = k.shape[0], k.shape[1]
    i = (torch.arange(R) if qpos is None else torch.as_tensor(qpos))[:, None]
    j = torch.arange(L)[None, :]
    seen = (j <= i) & ((i - j < size) | (j < keep))
    weights = torch.zeros(H, R, L, dtype=q.dtype)
    for hd in range(H):
        s = q[:, hd] @ k[:, hd // (H // G)].T * scale
        weights[hd] = torch.softmax(s.masked_fill(~seen, -math.inf), -1)
    mixed = torch.einsum("hg,gij->hij", talk, weights)
    return torch.stack([mixed[hd] @ v[:, hd // (H // G)] for hd in range(H)], 1)


def kept_first_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    factor = (rot.get("scaling") or {}).get("factor", 1.0)
    q = unit_rms((h @ w[p + "q"].T).view(T, H, d), eps) * w[p + "q.norm"]
    k = unit_rms((h @ w[p + "k"].T).view(T, G, d), eps) * w[p + "k.norm"]
    if rot["dims"]:
        q = rotate_half_split(q, pos, rot["dims"], rot["base"], factor)
        k = rotate_half_split(k, pos, rot["dims"], rot["base"], factor)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    out = kept_first_mixed(q, k, v, w[p + "talk"], m["scale"], m["mask"]["size"], m["mask"].get("keep_first") or 0)
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---- gated delta rule ---------------------------------------------------------------------------------
def short_convolution(z, taps):
    """z [T, C], taps [C, K]: y_t = sum_i taps[:, i] z_(t - (K-1) + i), zeros before the start."""
    T, K = z.shape[0], taps.shape[1]
    padded = torch.cat((torch.zeros(K - 1, z.shape[1], dtype=z.dtype), z), 0)
    return sum(padded[i:i + T] * taps[:, i] for i in range(K))


def delta_rule_scan(q, k, v, beta, g, S0=None, return_state=False):
    """q, k [T, H, d], v [T, H, dv], beta, g [T, H]; returns o [T, H, dv] (and the last state [H, d, dv])."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype) if S0 is None else S0.clone()
    o = torch.zeros_like(v)
    for t in range(T):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + torch.einsum("hd,hv->hdv", k[t], u)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return (o, S) if return_state else o


def delta_inputs(h, w, p, m):
    """q, k [T, G, d] (unit vectors, q times d^-1/2), v [T, H, dv], beta and g [T, H]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    return q, k, v, beta, g


def delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, dv = m["heads"], m["kv_heads"], m["vdim"]
    q, k, v, beta, g = delta_inputs(h, w, p, m)
    q, k = q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1)
    o = delta_rule_scan(q, k, v, beta, g)
    o = unit_rms(o, eps) * w[p + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---- routed feed-forward ------------------------------------------------------------------------------
def route(h, w, p, r):
    z = h @ w[p + "router"].T + w[p + "router.b"]
    top, chosen = torch.topk(z, r["top"], -1)
    return chosen, torch.softmax(top, -1)


def routed_ff(h, w, p, mlp):
    chosen, weights = route(h, w, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            pe = f"{p}e{e}."
            out[t] += a * ((silu(h[t] @ w[pe + "gate"].T) * (h[t] @ w[pe + "up"].T)) @ w[pe + "down"].T)
    return out


MIXERS = {"attention": pooled_window_attention, "attention_2": kept_first_attention, "delta": delta_mixer}


# ---- the model ----------------------------------------------------------------------------------------
def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence; with return_layers also the stream after every layer run."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        y = MIXERS[layer["type"]](x, w, p + "mix.", layer["mixer"], eps)
        x = x + m * unit_rms(y, eps) * w[p + "norm1"]
        if layer.get("mlp") is not None:
            y = routed_ff(x, w, p + "mlp.", layer["mlp"])
            x = x + m * unit_rms(y, eps) * w[p + "norm2"]
        streams.append(x.clone())
    logits = (unit_rms(x, eps) * w["final.norm"]) @ w["embed"].T
    return (logits, torch.stack(streams)) if return_layers else logits


def generate(cfg, w, prompt, n):
    """Greedy continuation, recomputing the whole sequence for every token."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(cfg, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
