"""Plain, slow restatement of the Silatar design in torch on the CPU — one function per mechanism, written from the
design's equations and sharing no code with the package.  It takes the config as the plain dict config.json holds and the
weights under their checkpoint names (as float tensors).

Silatar: a residual stream x [T, width]; every layer is  x += LN_b(mixer(LN_a(x)))  then  x += LN_d(ff(LN_c(x)))  with
weight-only layer norms; mixers are a latent (low-rank key/value) attention with interleaved, YaRN-stretched rotary
positions, or an mLSTM matrix memory with a stabilised exponential gate; feed-forwards are a dense erf-GELU layer or a
sigmoid-routed mixture of clamped gated experts with a gated shared expert; a span of layers may repeat; the logits are
soft-capped with tanh.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------------------------------- norms
def layer_norm(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = v.mean(-1, keepdim=True)
    var = ((v - mu) ** 2).mean(-1, keepdim=True)
    return (v - mu) / torch.sqrt(var + eps) * w


def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


# -------------------------------------------------------------------------------------------------------------- rotary
def rotary_frequencies(rot: dict, dtype=torch.float64):
    """Per-pair angular frequencies [dims/2] and the magnitude factor of cos / sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """v [T, ..., n]: the first rot.dims entries of the last axis are rotated pairwise (2i with 2i+1)."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot, torch.float64)
    ang = positions.to(torch.float64)[:, None] * f[None, :]                      # [T, dims/2]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [dims // 2]
    c, s = (torch.cos(ang) * mag).to(v.dtype).view(shape), (torch.sin(ang) * mag).to(v.dtype).view(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ----------------------------------------------------------------------------------------------------- latent attention
def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mixer: dict, eps: float,
                     positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Keys and values are expanded from a shared low-rank latent c; one rotated key part is shared by all heads."""
    T = h.shape[0]
    H, dn, dr, dv, r = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T).view(T, H, dn + dr)
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :r], eps) * w[p + "dkv.norm"]
    q_plain, q_rot, k_rot = q[..., :dn], q[..., dn:], down[:, r:]                 # k_rot [T, dr] is shared by the heads
    if mixer.get("rot"):
        q_rot, k_rot = rotate(q_rot, pos, mixer["rot"]), rotate(k_rot, pos, mixer["rot"])
    k_plain = (c @ w[p + "uk"].T).view(T, H, dn)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * mixer["scale"]      # [Tq, Tk]
        s = s.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, hd]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# --------------------------------------------------------------------------------------------------------------- mLSTM
def mlstm_cell(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gi: torch.Tensor, gf: torch.Tensor) -> torch.Tensor:
    """The recurrence alone.  q (already scaled), k [T, H, dk]; v [T, H, dv]; log gates gi, gf [T, H] → [T, H, dv].
    Per head: S [dk, dv], n [dk] and the running maximum m all start at 0."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=q.dtype)
        n = torch.zeros(dk, dtype=q.dtype)
        m = torch.zeros((), dtype=q.dtype)
        for t in range(T):
            m_new = torch.maximum(gf[t, hd] + m, gi[t, hd])
            a, b = torch.exp(gf[t, hd] + m - m_new), torch.exp(gi[t, hd] - m_new)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            m = m_new
            den = torch.maximum((n * q[t, hd]).sum().abs(), torch.exp(-m)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    return out


def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def mlstm(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mixer: dict, eps: float) -> torch.Tensor:
    """Matrix memory per head, token by token, then a unit-rms norm per head, a weight, an output gate and a projection."""
    T = h.shape[0]
    H, dk, dv, cap = mixer["heads"], mixer["dim"], mixer["vdim"], float(mixer["gate_cap"])
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    gi = capped(h @ w[p + "i"].T + w[p + "i.b"], cap)                                         # log input gate [T, H]
    gf = F.logsigmoid(capped(h @ w[p + "f"].T + w[p + "f.b"], cap))                           # log forget gate
    out = mlstm_cell(q, k, v, gi, gf)
    o = unit_rms(out, eps).reshape(T, H * dv) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    z = h @ w[p + "up"].T
    return (0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))) @ w[p + "down"].T


def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = (h @ w[p + "gate"].T).clamp(max=limit)
    u = (h @ w[p + "up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def routing(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, top: int):
    """→ chosen experts [T, top] and their weights: plain sigmoid scores, not renormalised."""
    s = torch.sigmoid(h @ w[p + "router"].T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    idx, val = routing(h, w, p, int(mlp["router"]["top"]))
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), val[t]):
            out[t] += expert(s * h[t:t + 1], w, f"{p}e{e}.", float(mlp["expert"]["limit"]))[0]   # weight on the INPUT
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)                                            # [T, 1]
        out = out + gate * expert(h, w, p + "shared.", float(mlp["shared"]["limit"]))
    return out


# --------------------------------------------------------------------------------------------------------------- model
def layer_runs(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop.get("times", 0)) <= 0:
        return list(range(n))
    a, b, k = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


def run_layer(x: torch.Tensor, cfg: dict, w: Dict[str, torch.Tensor], i: int) -> torch.Tensor:
    lc, eps, p = cfg["layers"][i], float(cfg["norm"]["eps"]), f"l{i}."
    h = layer_norm(x, w[p + "norm1"], eps)
    if lc["type"] == "latent_attention":
        y = latent_attention(h, w, p + "mix.", lc["mixer"], eps)
    elif lc["type"] == "mlstm":
        y = mlstm(h, w, p + "mix.", lc["mixer"], eps)
    else:
        raise ValueError(lc["type"])
    x = x + layer_norm(y, w[p + "norm1b"], eps)
    mlp = lc.get("mlp")
    if mlp is not None:
        h = layer_norm(x, w[p + "norm2"], eps)
        y = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
        x = x + layer_norm(y, w[p + "norm2b"], eps)
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence starting at position 0 (every run has fresh state).  `streams`, if a list,
    receives the residual stream after every layer run."""
    x = w["embed"][torch.tensor(tokens)]
    for i in layer_runs(cfg):
        x = run_layer(x, cfg, w, i)
        if streams is not None:
            streams.append(x.clone())
    z = layer_norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ w["head"].T
    cap = float(cfg["logit_softcap"])
    return cap * torch.tanh(z / cap)
