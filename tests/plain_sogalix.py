"""The Sogalix decoder written out plainly: float64, whole sequences, one function per mechanism.

Shares no code with the package; the package is tested against this.  ``cfg`` is the nested
dictionary of a config.json, ``W`` a dictionary name -> tensor (any element type; promoted here).

Notation: h input of a sub-layer [T, width]; p positions 0..T-1; H heads, d key size of a head,
e value size of a head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


# ----------------------------------------------------------------------------- small functions
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w.to(F) + b.to(F)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + z.clamp(min=0)


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    ap = softplus(torch.tensor(p, dtype=F))
    aq = 0.5 + softplus(torch.tensor(q, dtype=F))
    neg = z.clamp(max=0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(neg) - neg) + 0.5 * z)


def feed_forward(h, W, p):
    act = W[p + "act"].to(F)
    return xielu(h @ W[p + "up"].to(F).T, float(act[0]), float(act[1])) @ W[p + "down"].to(F).T


# ----------------------------------------------------------------------------- rotation
def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, n]: neighbours (2i, 2i+1), i < dims/2, of every head are turned by p * base^(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    a = positions.to(F)[:, None] * f[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- mixers
def general_delta(h, W, p, m, eps):
    """Per head a state S [d, d] (rows: key channels, columns: value channels), zero before position 0:
    S <- diag(w) S - (a * u)(u^T S) + k v^T with both products over the old S;  o = S^T r."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    lin = lambda n: (h @ W[p + n].to(F).T)
    r, k, v = (lin(n).view(T, H, d) for n in ("r", "k", "v"))
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(lin("w1")) @ W[p + "w2"].to(F).T + W[p + "w0"].to(F))).view(T, H, d)
    a = torch.sigmoid(lin("a") + W[p + "a.b"].to(F)).view(T, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=F)
    o = torch.zeros(T, H, d, dtype=F)
    for t in range(T):
        uS = torch.einsum("hc,hce->he", u[t], S)
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hc,hce->he", r[t], S)
    o = rms_unit(o, eps).reshape(T, H * d) * W[p + "norm"].to(F) * torch.sigmoid(lin("g"))
    return o @ W[p + "o"].to(F).T


def query_temperature(positions, q_temp):
    if not q_temp:
        return torch.ones(positions.shape[0], dtype=F)
    return 1.0 + float(q_temp["coef"]) * torch.log(torch.floor((positions.to(F) + 1) / int(q_temp["every"])) + 1.0)


def sink_attention(h, W, p, m):
    """Causal softmax attention without rotation whose denominator has one more term of score 0."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ W[p + "q"].to(F).T).view(T, H, d) * query_temperature(pos, m.get("q_temp"))[:, None, None]
    k = (h @ W[p + "k"].to(F).T).view(T, G, d)
    v = (h @ W[p + "v"].to(F).T).view(T, G, e)
    causal = pos[None, :] <= pos[:, None]
    out = torch.zeros(T, H, e, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        ex = torch.where(causal, torch.exp(s), torch.zeros_like(s))
        out[:, hd] = (ex / (1.0 + ex.sum(-1, keepdim=True))) @ v[:, g]
    return out.reshape(T, H * e) @ W[p + "o"].to(F).T


def latent_and_rotated_key(h, W, p, m, eps):
    """What a latent-attention layer with keys of its own keeps per position: (c [T, kv_rank], rotated key part [T, rot_dim])."""
    T = h.shape[0]
    kv = h @ W[p + "dkv"].to(F).T
    R = m["kv_rank"]
    c = rms_unit(kv[:, :R], eps) * W[p + "dkv.norm"].to(F)
    kr = rotate_pairs(kv[:, None, R:], torch.arange(T), int(m["rot"]["dims"]), float(m["rot"]["base"]))[:, 0]
    return c, kr


def latent_attention(h, W, p, m, eps, kept):
    """``kept``: (c, rotated key part) of this layer or of the layer it reads."""
    T = h.shape[0]
    H, d, n, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_unit(h @ W[p + "dq"].to(F).T, eps) * W[p + "dq.norm"].to(F)
    q = (cq @ W[p + "uq"].to(F).T).view(T, H, d + n)
    q_plain = q[..., :d]
    q_rot = rotate_pairs(q[..., d:], pos, int(m["rot"]["dims"]), float(m["rot"]["base"]))
    c, kr = kept
    k_plain = (c @ W[p + "uk"].to(F).T).view(T, H, d)
    v = (c @ W[p + "uv"].to(F).T).view(T, H, e)
    gate = torch.sigmoid(h @ W[p + "g"].to(F).T)            # [T, H]
    causal = pos[None, :] <= pos[:, None]
    out = torch.zeros(T, H, e, dtype=F)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ kr.T) * float(m["scale"])
        s = torch.where(causal, s, torch.full_like(s, -math.inf))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, hd] * gate[:, hd:hd + 1]
    return out.reshape(T, H * e) @ W[p + "o"].to(F).T


# ----------------------------------------------------------------------------- the model
def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """float64 logits [T, vocab] of one whole sequence; ``layers_out`` collects the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    norm = lambda x, name: layer_norm(x, W[name], W[name + ".b"], eps)
    x = norm(W["embed"].to(F)[torch.tensor(tokens)], "embed.norm")
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm(x, p + "norm1")
        m = L["mixer"]
        if L["type"] == "general_delta":
            y = general_delta(h, W, p + "mix.", m, eps)
        elif L["type"] == "attention":
            y = sink_attention(h, W, p + "mix.", m)
        elif L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_and_rotated_key(h, W, p + "mix.", m, eps)
                src = i
            y = latent_attention(h, W, p + "mix.", m, eps, kept[src])
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp") is not None:
            x = x + feed_forward(norm(x, p + "norm2"), W, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, "final.norm") @ W["head"].to(F).T


# ----------------------------------------------------------------------------- model folders of random weights
def tensor_shapes(cfg: dict, decay_rank: int = 6) -> Dict[str, tuple]:
    V, Wd = cfg["vocab"], cfg["width"]
    out = {"embed": (V, Wd), "head": (V, Wd)}
    for n in ("embed.norm", "final.norm"):
        out[n], out[n + ".b"] = (Wd,), (Wd,)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        for n in ("norm1",) + (("norm2",) if L.get("mlp") else ()):
            out[p + n], out[p + n + ".b"] = (Wd,), (Wd,)
        q = p + "mix."
        if L["type"] == "general_delta":
            n = m["heads"] * m["dim"]
            out.update({q + "r": (n, Wd), q + "k": (n, Wd), q + "v": (n, Wd), q + "g": (n, Wd), q + "a": (n, Wd), q + "a.b": (n,),
                        q + "w1": (decay_rank, Wd), q + "w2": (n, decay_rank), q + "w0": (n,), q + "norm": (n,), q + "o": (Wd, n)})
        elif L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({q + "q": (H * d, Wd), q + "k": (G * d, Wd), q + "v": (G * e, Wd), q + "o": (Wd, H * e)})
        else:
            H, d, n, e, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({q + "dq": (Q, Wd), q + "dq.norm": (Q,), q + "uq": (H * (d + n), Q), q + "uk": (H * d, R), q + "uv": (H * e, R),
                        q + "g": (H, Wd), q + "o": (Wd, H * e)})
            if m.get("kv_from") is None:
                out.update({q + "dkv": (R + n, Wd), q + "dkv.norm": (R,)})
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            out.update({p + "mlp.up": (ff, Wd), p + "mlp.down": (Wd, ff), p + "mlp.act": (2,)})
    return out


def random_weights(cfg: dict, seed: int, dtype=torch.float32, decay_rank: int = 6) -> Dict[str, torch.Tensor]:
    """Weights drawn so that no mechanism drowns: matrices N(0, 1.5^2 / fan_in), norm weights around one with small
    biases, decays and removal rates spread over their ranges."""
    gen = torch.Generator().manual_seed(seed)
    rand = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
    uni = lambda lo, hi, *s: lo + (hi - lo) * torch.rand(*s, generator=gen, dtype=torch.float32)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg, decay_rank).items()):
        last = name.split(".")[-1]
        if name == "embed":
            t = rand(*shape) * 0.7
        elif last == "b" and name.endswith("a.b"):
            t = uni(-2.0, 2.0, *shape)
        elif last == "b":
            t = 0.1 * rand(*shape)
        elif last in ("norm1", "norm2", "norm"):
            t = 1 + 0.2 * rand(*shape)
        elif last == "w0":
            t = uni(-4.0, 3.0, *shape)
        elif last == "w2":
            t = rand(*shape) * 1.5
        elif last == "act":
            t = uni(-1.0, 1.0, *shape)
        else:
            t = rand(*shape) * (1.5 / math.sqrt(shape[-1]))
        out[name] = t.to(dtype)
    return out


def write_model(folder, cfg: dict, seed: int, dtype=torch.float32, weights=None):
    """A model folder (config.json, model.safetensors); returns the weights as stored."""
    import json
    from pathlib import Path
    from pytriton_llama_b200.weights import write_file      # only the file format comes from the package
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    W = weights if weights is not None else random_weights(cfg, seed, dtype)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_file(folder / "model.safetensors", W)
    return W


def delta(heads, dim):
    return {"heads": heads, "dim": dim}


def attention(heads, kv_heads, dim, vdim, scale, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(vocab, width, layers, eps=1e-5):
    return {"architecture": "Sogalix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# A reader of another layer's latent two layers on; value heads larger than key heads; a temperature that steps every 5
# positions; a delta layer with a feed-forward and an attention layer without.
TINY_A = config(97, 48, [
    layer("latent_attention", latent(3, 16, 8, 24, 20, 28, 0.2, 1000.0), dense(40)),
    layer("general_delta", delta(3, 8), dense(24)),
    layer("attention", attention(4, 2, 16, 24, 0.3, q_temp=(0.4, 5)), None),
    layer("latent_attention", latent(3, 16, 8, 24, 20, 28, 0.25, 1000.0, kv_from=0), None),
], eps=1e-5)
# One wide delta head (more rows than a warp's packet); as many kv heads as heads and no temperature; a latent layer
# with a single head whose rotated part is larger than its plain part.
TINY_B = config(70, 64, [
    layer("general_delta", delta(1, 40), None),
    layer("attention", attention(6, 6, 16, 16, 0.35), dense(72)),
    layer("latent_attention", latent(1, 8, 24, 40, 12, 10, 0.3, 50.0), dense(32)),
    layer("general_delta", delta(2, 32), None),
], eps=3e-4)
# One kv head for three query heads with a temperature every position; two readers of one latent; odd sizes.
TINY_C = config(50, 32, [
    layer("attention", attention(3, 1, 24, 8, 0.3, q_temp=(1.0, 1)), dense(48)),
    layer("latent_attention", latent(2, 12, 4, 10, 6, 14, 0.4, 300.0), None),
    layer("general_delta", delta(4, 4), None),
    layer("latent_attention", latent(5, 6, 4, 6, 6, 8, 0.5, 300.0, kv_from=1), dense(16)),
    layer("latent_attention", latent(2, 8, 4, 16, 6, 9, 0.3, 300.0, kv_from=1), None),
])
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
