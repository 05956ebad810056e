"""A plain, slow Tudasun: one function per mechanism, whole sequences at once, no cache.

Written from the design's equations with torch on the CPU; it shares no code with the engine and
is the oracle of the tests.  Notation: x is the residual stream [T, W]; matrices are stored
[out, in] and applied as ``h @ W.T``; positions are 0 .. T-1; rms(y) = y / sqrt(mean(y^2) + eps).

    embedding        x = E[token]
    layer            h = n1(x);  x = x + n1b(mixer(h) * sigmoid(R1 h + r1))
                     h = n2(x);  x = x + n2b(ff(h) * sigmoid(R2 h + r2))        (if the layer has a feed-forward)
                     e = T[token, i d : (i+1) d];  y = P (gelu_tanh(G x) * e);  x = x + rms(y) * w_side
    norm             n(x) = rms(x) * (1 + w)
    gla              q = W_q h / sqrt(dim), k = W_k h, v = W_v h; decay a = sigmoid(A2 (A1 h) + b)^(1/tau) per key channel;
                     S_t = diag(a_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;  per head rms(o) * w;  times silu(W_g h);  W_o
    hgrn2            q = silu(W_q h), v = W_v h;  f = l + (1 - l) sigmoid(W_f h + b);
                     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T;  o_t = S_t^T q_t;  per head rms(o) * w;  W_o
    latent attention [c ; kr] = W_dkv h;  c = rms(c) * w_c;  kr rotated (interleaved pairs), shared by the heads;
                     k_h = [W_uk c ; kr], v_h = W_uv c, q_h = [unrotated ; rotated];  causal softmax whose
                     denominator also holds exp(sink_h);  W_o.  A layer with kv_from j uses layer j's c and kr.
    dense ff         W_down polynorm(W_up h);  polynorm(z) = a rms(z) + b rms(z^2) + c rms(z^3) + e
    routed ff        s = softmax(W_r h) over experts and identity experts; chosen by s + correction among the best
                     groups; weights s / (sum + 1e-20); experts W_down (silu(W_gate h) * W_up h), identity experts h;
                     plus sigmoid(w_sg . h) * shared(h)
    output           logits = H n_final(x);  logits = cap tanh(logits / cap)
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


def offset_norm(x, w, eps):
    """rms(x) * (1 + w): the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_interleaved(t, positions, dims, base):
    """t [T, n, d]: the pairs (2i, 2i + 1) of the first ``dims`` elements turn by position * base^(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=t.dtype)
    a = positions.to(t.dtype)[:, None] * base ** (-2.0 * i / dims)[None, :]
    cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = t[..., 0:dims:2], t[..., 1:dims:2]
    out = t.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ---- the two recurrences ---------------------------------------------------------------------------
def decayed_outer_scan(q, k, v, decay):
    """q, k, decay [T, H, dk], v [T, H, dv]:  S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, S_(-1) = 0."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out)


def gla_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    decay = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).view(T, H, dk)
    o = decayed_outer_scan(q, k, v, decay)
    o = unit_rms(o, eps) * w[p + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def hgrn2_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w[p + "f"].T + w[p + "f.b"])).view(T, H, dk)
    o = decayed_outer_scan(q, 1.0 - f, v, f)
    o = unit_rms(o, eps) * w[p + "norm"]
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ---- latent attention ----------------------------------------------------------------------------------
def latent_rows(h, w, p, m, eps):
    """What the layer caches: the normalised latent [T, rank] and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    rank, dr = m["kv_rank"], m["rot_dim"]
    ckr = h @ w[p + "dkv"].T
    c = unit_rms(ckr[:, :rank], eps) * w[p + "dkv.norm"]
    kr = rotate_interleaved(ckr[:, None, rank:], torch.arange(T), m["rot"]["dims"], m["rot"]["base"])[:, 0]
    return c, kr


def latent_attention_mixer(h, w, p, m, rows):
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = rows
    q = (h @ w[p + "q"].T).view(T, H, d + dr)
    qr = rotate_interleaved(q[..., d:], torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    kn = (c @ w[p + "uk"].T).view(T, H, d)
    val = (c @ w[p + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q[..., :d], kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    s = s.masked_fill(~causal, -math.inf)
    sink = w[p + "sink"][:, None, None].expand(H, T, 1)
    prob = torch.softmax(torch.cat((s, sink), -1), -1)[..., :T]        # the sink takes its share and gives nothing
    o = torch.einsum("hij,jhd->ihd", prob, val).reshape(T, H * dv)
    return o @ w[p + "o"].T


# ---- feed-forwards ---------------------------------------------------------------------------------------
def polynorm(z, coef, eps):
    a, b, c, e = coef
    return a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e


def dense_ff(h, w, p, eps):
    return polynorm(h @ w[p + "up"].T, w[p + "act"], eps) @ w[p + "down"].T


def gated_expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, r):
    """(chosen [T, top], weights [T, top]) of the router over ``experts + identity`` outputs."""
    n, top = r["experts"] + r["identity"], r["top"]
    s = torch.softmax(h @ w[p + "router"].T, -1)
    choice = s + w[p + "correction"]
    groups = r.get("groups")
    if groups is not None:
        per = n // groups["count"]
        best = choice.view(-1, groups["count"], per).max(-1).values
        kept = best.topk(groups["keep"], -1).indices
        allow = torch.zeros_like(best, dtype=torch.bool).scatter(1, kept, True)
        choice = choice.masked_fill(~allow.repeat_interleave(per, 1), -math.inf)
    chosen = choice.topk(top, -1).indices
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20)


def routed_ff(h, w, p, mlp):
    r = mlp["router"]
    chosen, weights = route(h, w, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            y = h[t] if e >= r["experts"] else gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
            out[t] += g * y
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_expert(h, w, p + "shared.")
    return out


# ---- the per-layer token input -------------------------------------------------------------------------
def token_side(x, tokens, w, i, dim, eps):
    p = f"l{i}.side."
    e = w["side.embed"][tokens, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return unit_rms(y, eps) * w[p + "norm"]


# ---- the model ---------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"][tokens]
    side = cfg.get("token_side")
    cached, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = offset_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "gla":
            a = gla_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "hgrn2":
            a = hgrn2_mixer(h, w, p + "mix.", m, eps)
        else:
            owner = m.get("kv_from")
            if owner is None:
                cached[i] = latent_rows(h, w, p + "mix.", m, eps)
                owner = i
            a = latent_attention_mixer(h, w, p + "mix.", m, cached[owner])
        a = a * torch.sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"])
        x = x + offset_norm(a, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = offset_norm(x, w[p + "norm2"], eps)
            f = dense_ff(h, w, p + "mlp.", eps) if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp)
            f = f * torch.sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"])
            x = x + offset_norm(f, w[p + "norm2b"], eps)
        if side is not None:
            x = x + token_side(x, tokens, w, i, side["dim"], eps)
        after.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if return_layers else logits


def generate(cfg, w, prompt, n):
    """Greedy continuation of ``prompt`` by n tokens (lowest index wins ties), whole sequence each time."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(cfg, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
