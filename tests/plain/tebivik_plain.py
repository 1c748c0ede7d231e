"""Plain, slow implementation of the Tebivik decoder: the oracle of its tests.

Whole sequences, no cache, no state carried between calls, Python loops over time where the design has a
recurrence, one function for each mechanism.  Nothing here imports the engine's package; the configuration and
the weights are read by this file's own code.

Notation.  T tokens, width D.  Linear weights are stored [out, in] and applied as ``x @ W.T``.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# ----------------------------------------------------------------------------- files
def load_config(model_dir) -> dict:
    return json.loads((Path(model_dir) / "config.json").read_text())


def load_weights(model_dir, dtype=torch.float64) -> dict[str, torch.Tensor]:
    """model.safetensors read by hand: 8 bytes of header length, a JSON header, then the tensors' bytes."""
    raw = (Path(model_dir) / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64}
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        lo, hi = rec["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=kinds[rec["dtype"]]).reshape(rec["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return out


# ------------------------------------------------------------------------------------- parts
def group_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, groups: int) -> torch.Tensor:
    """The last axis is cut into ``groups`` equal consecutive parts; each part is divided by
    sqrt(mean(part^2) + eps); the whole is then multiplied by w."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(x.shape) * w


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return group_rms_norm(x, w, eps, 1)


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h: [T, D]; w: [D, taps].  y_t = sum_j w[:, j] * h_(t - taps + 1 + j), h = 0 at negative times."""
    T, taps = h.shape[0], w.shape[1]
    y = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * h[s]
    return y


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x: [T, ..., d].  The first ``dims`` entries of the last axis are rotated in pairs (2i, 2i+1) by the angle
    position * base^(-2i/dims); entries from ``dims`` on are copied."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]  # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(ang).reshape(shape).to(x.dtype), torch.sin(ang).reshape(shape).to(x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def hgrn2(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Gated linear recurrence whose forget gate also says how much is written.  Per head, with state S [dim, vdim]
    starting at zero:  S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T ;  o_t = S_t^T q_t."""
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = torch.nn.functional.silu(h @ w[p + "q"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    lower = w[p + "lower"]
    f = lower + (1 - lower) * torch.sigmoid(h @ w[p + "f"].T + w[p + "f.b"])
    f = f.reshape(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o, w[p + "norm"], eps)  # per head over vdim, one weight for all heads
    return o.reshape(T, H * dv) @ w[p + "o"].T


def latent_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Attention whose queries, keys and values come out of low-rank latents; one rotated key part is shared by
    all heads; the softmax's denominator holds one more term exp(sink_h) to which no key and no value row belong."""
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(T)
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_n, q_r = q[..., :dn], q[..., dn:]
    ckv = h @ w[p + "dkv"].T
    c = rms_norm(ckv[:, :rank], w[p + "dkv.norm"], eps)
    k_r = ckv[:, rank:]  # [T, dr], not normed, one for all heads
    rot = m["rot"]
    q_r = rotate_pairs(q_r, pos, rot["base"], rot["dims"])
    k_r = rotate_pairs(k_r, pos, rot["base"], rot["dims"])
    k_n = (c @ w[p + "uk"].T).reshape(T, H, dn)
    val = (c @ w[p + "uv"].T).reshape(T, H, dv)
    s = (torch.einsum("thd,shd->hts", q_n, k_n) + torch.einsum("thd,sd->hts", q_r, k_r)) * m["scale"]
    mask = pos[None, :] <= pos[:, None]  # [t, s]: key s visible to query t
    s = s.masked_fill(~mask[None], float("-inf"))
    sink = w[p + "sink"].to(s.dtype)  # [H]
    big = torch.maximum(s.max(dim=-1).values, sink[:, None])  # [H, T]
    e = torch.exp(s - big[..., None])
    prob = e / (e.sum(dim=-1) + torch.exp(sink[:, None] - big))[..., None]
    out = torch.einsum("hts,shd->thd", prob, val)
    return out.reshape(T, H * dv) @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    a = torch.relu(h @ w[p + "up"].T + w[p + "up.b"]) ** 2
    return a @ w[p + "down"].T + w[p + "down.b"]


MIXERS = {"hgrn2": hgrn2, "latent_attention": latent_attention}


def layer(x: torch.Tensor, cfg: dict, w: dict, i: int) -> torch.Tensor:
    spec, p = cfg["layers"][i], f"l{i}."
    eps, groups, mult = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["residual_mult"]
    h = group_rms_norm(x, w[p + "norm1"], eps, groups)
    h = h + causal_conv(h, w[p + "canon1"])
    y = MIXERS[spec["type"]](h, w, p + "mix.", spec["mixer"], eps)
    x = x + mult * group_rms_norm(y, w[p + "norm1b"], eps, groups)
    if spec["mlp"] is not None:
        y = dense_ff(group_rms_norm(x, w[p + "norm2"], eps, groups), w, p + "mlp.")
        x = x + mult * group_rms_norm(y, w[p + "norm2b"], eps, groups)
    return x


def layer_order(cfg: dict) -> list[tuple[int, int | None]]:
    """(layer, number of the pass whose first layer it is, or None) in the order of execution."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg: dict, w: dict, tokens, residuals: list | None = None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence.  ``residuals`` collects the stream after every layer run."""
    x0 = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)] * cfg["embedding"]["scale"]
    x = x0
    for i, first_of_pass in layer_order(cfg):
        if first_of_pass is not None:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][first_of_pass]
        x = layer(x, cfg, w, i)
        if residuals is not None:
            residuals.append(x)
    x = group_rms_norm(x, w["final.norm"], cfg["norm"]["eps"], cfg["norm"]["groups"])
    return x @ w["embed"].T


def greedy_generate(cfg: dict, w: dict, prompt, n_new: int) -> list[int]:
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(cfg, w, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
