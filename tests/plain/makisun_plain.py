"""A plain, slow Makisun: one function per mechanism, float64 on the CPU, token by token where the design is a recurrence.

It shares nothing with the package: its own config reading (plain dictionaries), its own safetensors reader, its own
formulas.  ``forward`` runs whole sequences; the tests compare the engine's logits, however its steps were cut, with these.

Notation: h [T, D] rows of one sequence; W [out, in] applied as ``h @ W.T``; P maps tensor names to float64 tensors.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64


def read_safetensors(path) -> dict:
    """name -> float64 tensor (integers stay integers): 8 bytes of header length, a JSON header, then the data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    types = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64, "I32": torch.int32,
             "I64": torch.int64}
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=types[meta["dtype"]]).reshape(meta["shape"])
        out[name] = t.to(F64) if t.is_floating_point() else t
    return out


def rms_divide(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The layer norm of this design: the stored weight is an offset from one."""
    return rms_divide(x, eps) * (1.0 + w)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def silu(z):
    return z * torch.sigmoid(z)


def rotate_half(x, positions, base, dims):
    """x [T, heads, d]: entry i < dims/2 is paired with entry i + dims/2; entries from ``dims`` on pass unchanged."""
    half = dims // 2
    if half == 0:
        return x
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = positions.to(F64)[:, None, None] * f[None, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def window_attention(h, P, p, m, eps):
    """Grouped-query softmax attention over the last ``mask.size`` positions, normed and partly rotated q and k, and a
    sigmoid gate per head on the output."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ P[p + "q"].T).view(T, H, d)
    k = (h @ P[p + "k"].T).view(T, G, d)
    v = (h @ P[p + "v"].T).view(T, G, dv)
    q = rms_divide(q, eps) * P[p + "q.norm"]
    k = rms_divide(k, eps) * P[p + "k.norm"]
    pos = torch.arange(T)
    q = rotate_half(q, pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half(k, pos, m["rot"]["base"], m["rot"]["dims"])
    gate = torch.sigmoid(h @ P[p + "g"].T)  # [T, H]
    span = m["mask"]["size"]
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        lo = max(0, i - span + 1)
        for a in range(H):
            g = a // (H // G)
            s = (k[lo:i + 1, g] @ q[i, a]) * m["scale"]
            w = torch.softmax(s, dim=0)
            out[i, a] = w @ v[lo:i + 1, g]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ P[p + "o"].T


def gated_linear_attention(h, P, p, m, eps):
    """S <- diag(alpha) S + k v^T, o = S^T q, with a per-key-channel decay alpha = sigmoid(z)^(1/tau)."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ P[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ P[p + "k"].T).view(T, H, d)
    v = (h @ P[p + "v"].T).view(T, H, dv)
    z = (h @ P[p + "a1"].T) @ P[p + "a2"].T + P[p + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / m["tau"])).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_divide(o, eps) * P[p + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ P[p + "g"].T)) @ P[p + "o"].T


def parallel_mixer(h, P, p, m, eps):
    left = window_attention(h, P, p + "left.", m["left"], eps)
    right = gated_linear_attention(h, P, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def wkv_mixer(h, P, p, m, eps):
    """Time mixing with a data-dependent decay: every projection reads its own blend of the token and the one before;
    the current token reaches the output through the bonus u, older ones through the decayed state."""
    T, D = h.shape
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, D, dtype=F64), h[:-1]], dim=0)

    def blend(s):
        return h + (prev - h) * P[p + "mu." + s]

    r = (blend("r") @ P[p + "r"].T).view(T, H, d)
    k = (blend("k") @ P[p + "k"].T).view(T, H, d)
    v = (blend("v") @ P[p + "v"].T).view(T, H, d)
    gate = silu(blend("g") @ P[p + "g"].T)
    w = torch.exp(-torch.exp(torch.tanh(blend("w") @ P[p + "w1"].T) @ P[p + "w2"].T + P[p + "w0"])).view(T, H, d)
    u = P[p + "u"]
    S = torch.zeros(H, d, d, dtype=F64)
    o = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = w[t][:, :, None] * S + kv
    o = rms_divide(o, eps).reshape(T, H * d) * P[p + "norm"]
    return (o * gate) @ P[p + "o"].T


def dense_mlp(h, P, p):
    return gelu_erf(h @ P[p + "up"].T) @ P[p + "down"].T


def expert(h, P, p):
    return relu_squared(h @ P[p + "up"].T) @ P[p + "down"].T


def router_logits(h, P, p):
    return h @ P[p + "router"].T + P[p + "router.b"]


def mixture_of_experts(h, P, p, mlp, forced=None):
    """``forced`` [T, top] replaces the choice (the tests hand over the engine's, where two logits nearly tie)."""
    z = router_logits(h, P, p)
    top = mlp["router"]["top"]
    chosen = torch.topk(z, top, dim=-1).indices if forced is None else forced.to(torch.int64)
    weights = torch.softmax(torch.gather(z, 1, chosen), dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            out[t] += weights[t, j] * expert(h[t:t + 1], P, f"{p}e{int(chosen[t, j])}.")[0]
    if mlp.get("shared") is not None:
        out = out + expert(h, P, p + "shared.")
    return out, z, chosen


def forward(config: dict, P: dict, tokens, forced_routing=None):
    """logits [T, vocab], the residual stream after every layer [L, T, D], router logits per routed layer."""
    eps = config["norm"]["eps"]
    x = P["embed"][torch.as_tensor(tokens, dtype=torch.int64)] * config["embedding"]["scale"]
    after, routers, n_routed = [], [], 0
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        h = norm_one_plus(x, P[p + "norm1"], eps)
        mixer = {"wkv": wkv_mixer, "parallel": parallel_mixer}[L["type"]]
        x = x + P[p + "ls1"] * mixer(h, P, p + "mix.", L["mixer"], eps)
        if L.get("mlp") is not None:
            h = norm_one_plus(x, P[p + "norm2"], eps)
            if L["mlp"]["kind"] == "dense":
                y = dense_mlp(h, P, p + "mlp.")
            else:
                forced = None if forced_routing is None else forced_routing[n_routed]
                y, z, chosen = mixture_of_experts(h, P, p + "mlp.", L["mlp"], forced)
                routers.append((z, chosen))
                n_routed += 1
            x = x + P[p + "ls2"] * y
        after.append(x.clone())
    logits = norm_one_plus(x, P["final.norm"], eps) @ P["head"].T
    return logits, torch.stack(after), routers
