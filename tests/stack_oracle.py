"""Plain, slow restatement of the Kozusun design in torch fp32 on the CPU — one function per mechanism, written from the
design's equations and sharing no code with the package.  It takes the config as the plain dict config.json holds and the
weights under their checkpoint names.

Notation: x residual stream [T, width]; x0 embedding output; m residual multiplier; eps the norm's epsilon;
rms(v) = v / sqrt(mean(v²) + eps).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def norm_zero_centred(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Block / final norm: the stored weight is centred on zero."""
    return rms(v, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sees(i: int, j: int, size: int, keep_first: int) -> bool:
    """Query position i sees key position j."""
    return j <= i and (i - j < size or j < keep_first)


def embed(tokens: List[int], table: torch.Tensor, scale: float) -> torch.Tensor:
    return table[torch.tensor(tokens)] * scale


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mixer: dict) -> torch.Tensor:
    """Gated sliding-window attention with kept first tokens over a whole sequence (positions 0 … T-1), key by key."""
    T = h.shape[0]
    H, G, dk, dv = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    size, keep = mixer["mask"]["size"], mixer["mask"]["keep_first"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)                        # [T, H]
    out = torch.zeros(T, H, dv)
    for i in range(T):
        js = [j for j in range(T) if sees(i, j, size, keep)]
        for hd in range(H):
            kv = hd // (H // G)
            s = torch.stack([(q[i, hd] * k[j, kv]).sum() for j in js]) * mixer["scale"]
            pr = torch.softmax(s, 0)
            out[i, hd] = sum(pr[n] * v[j, kv] for n, j in enumerate(js)) * gate[i, hd]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def token_side(x: torch.Tensor, tokens: List[int], layer: int, w: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    d, p = cfg["token_side"]["dim"], f"l{layer}.side."
    e = w["side.embed"][torch.tensor(tokens)][:, layer * d:(layer + 1) * d]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return cfg["residual_mult"] * rms(y, cfg["norm"]["eps"]) * w[p + "norm"]


def layer_order(cfg: dict) -> List[tuple]:
    """(layer, does a loop pass start here) for every layer run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    out = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        out += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return out + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence fed whole."""
    w = {k: v.float() for k, v in w.items()}
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x0 = embed(tokens, w["embed"], cfg["embedding"]["scale"])
    x = x0.clone()
    for i, starts_pass in layer_order(cfg):
        lc = cfg["layers"][i]
        if starts_pass:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T
        h = norm_zero_centred(x, w[f"l{i}.norm1"], eps)
        y = attention(h, w, f"l{i}.mix.", lc["mixer"])
        if lc["mlp"] is not None:
            y = y + feed_forward(h, w, f"l{i}.mlp.")
        x = x + m * y
        if "token_side" in cfg:
            x = x + token_side(x, tokens, i, w, cfg)
        if streams is not None:
            streams.append(x.clone())
    return norm_zero_centred(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> tuple:
    """→ (tokens, top-2 margins): n_new greedy tokens, re-running the whole sequence for every one."""
    toks, out, margins = list(prompt), [], []
    for _ in range(n_new):
        lg = forward(cfg, w, toks)[-1]
        top = torch.topk(lg, 2).values
        margins.append(float(top[0] - top[1]))
        out.append(int(lg.argmax()))
        toks.append(out[-1])
    return out, margins


# ------------------------------------------------------------------------------------------------ test material
def make_config(width=64, vocab=96, layers=None, loop=None, side_dim=8, embed_scale=3.0, residual_mult=0.4,
                eps=1e-5) -> dict:
    """A config dict of the design.  `layers`: list of dicts {heads, kv_heads, dim, vdim, size, keep_first, ff}; ff None =
    no feed-forward."""
    layers = layers or [dict(heads=4, kv_heads=2, dim=16, vdim=8, size=6, keep_first=2, ff=48)] * 2
    cfg = {"architecture": "Kozusun", "embedding": {"scale": embed_scale}, "layers": [], "norm": {"eps": eps},
           "residual_mult": residual_mult, "vocab": vocab, "width": width}
    for L in layers:
        cfg["layers"].append({
            "type": "attention",
            "mixer": {"dim": L["dim"], "heads": L["heads"], "kv_heads": L["kv_heads"], "vdim": L["vdim"],
                      "scale": L.get("scale", 1.0 / math.sqrt(L["dim"])),
                      "mask": {"keep_first": L["keep_first"], "size": L["size"]}},
            "mlp": None if L.get("ff") is None else {"ff": L["ff"], "kind": "dense"}})
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if side_dim:
        cfg["token_side"] = {"dim": side_dim}
    return cfg


def make_weights(cfg: dict, seed: int = 0, std: float = 0.08) -> Dict[str, torch.Tensor]:
    """Random bf16 checkpoint of the design: matrices N(0, std·√(64/in)), zero-centred norm weights and biases N(0, 0.1),
    the side norm's plain weight around 1."""
    g = torch.Generator().manual_seed(seed)
    W, V, n = cfg["width"], cfg["vocab"], len(cfg["layers"])

    def mat(o, i):
        return (torch.randn(o, i, generator=g) * std * math.sqrt(64.0 / i)).to(torch.bfloat16)

    def vec(k, centre=0.0):
        return (centre + torch.randn(k, generator=g) * 0.1).to(torch.bfloat16)

    w = {"embed": mat(V, W), "final.norm": vec(W), "head": mat(V, W)}
    if cfg.get("loop"):
        w["loop.in"] = mat(W, 2 * W)
    if "token_side" in cfg:
        w["side.embed"] = (torch.randn(V, n * cfg["token_side"]["dim"], generator=g)).to(torch.bfloat16)
    for i, lc in enumerate(cfg["layers"]):
        mx, p = lc["mixer"], f"l{i}."
        w[p + "norm1"] = vec(W)
        for nm, rows in (("q", mx["heads"] * mx["dim"]), ("k", mx["kv_heads"] * mx["dim"]), ("v", mx["kv_heads"] * mx["vdim"])):
            w[p + "mix." + nm] = mat(rows, W)
            w[p + "mix." + nm + ".b"] = vec(rows)
        w[p + "mix.g"] = mat(mx["heads"], W)
        w[p + "mix.o"] = mat(W, mx["heads"] * mx["vdim"])
        if lc["mlp"] is not None:
            ff = lc["mlp"]["ff"]
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, W), mat(ff, W), mat(W, ff)
        if "token_side" in cfg:
            d = cfg["token_side"]["dim"]
            w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"] = mat(d, W), mat(W, d), vec(W, 1.0)
    return w
