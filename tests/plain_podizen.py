"""The Podizen decoder written out plainly: float64, whole sequences, one function per mechanism.

Shares no code with the package; the package is tested against this.  ``cfg`` is the nested
dictionary of a config.json, ``W`` a dictionary name -> tensor (any element type; promoted here).

Notation: h input of a sub-layer [T, width]; positions 0..T-1; H query heads, G key/value heads,
d query/key head size, e value head size, n window size, P pooled block length.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w.to(F)


def silu(z):
    return z * torch.sigmoid(z)


def lin(h, W, name):
    return h @ W[name].to(F).T


# ----------------------------------------------------------------------------- rotation of half-split pairs
def rotate_halves(x: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, d]: entry i of the first ``dims`` of a head is paired with entry i + dims/2 and the
    pair is turned by position * base^(-2i/dims)."""
    if not rot:
        return x
    n, base = int(rot["dims"]), float(rot["base"])
    half = n // 2
    f = base ** (-2.0 * torch.arange(half, dtype=F) / n)
    a = torch.arange(x.shape[0], dtype=F)[:, None] * f[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:n]
    out[..., :half] = u * c - v * s
    out[..., half:n] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- softmax attention
def distance_slopes(H: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (a + 1) / H) for a in range(H)], dtype=F)


def softmax_attention(q, k, v, scale: float, window: int, pool: int = 0, slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].  Query i sees the keys j with 0 <= i - j < window
    (window 0: every j <= i).  With ``pool`` = P > 0 it also sees, for every block b of P positions whose last
    position bP + P - 1 is at most i - window, the mean key and mean value of the block; one softmax over both.
    ``slopes`` [H]: slope * (i - j) is taken off the score of a token."""
    T, H, d = q.shape
    G, e = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, e, dtype=F)
    nb = T // pool if pool else 0
    if nb:
        kb = k[:nb * pool].view(nb, pool, G, d).mean(dim=1)
        vb = v[:nb * pool].view(nb, pool, G, e).mean(dim=1)
    for i in range(T):
        lo = max(0, i - window + 1) if window else 0
        nvis = 0
        if nb and window:
            nvis = min(nb, max(0, (i - window + 1) // pool))     # blocks with bP + P - 1 <= i - window
        for a in range(H):
            g = a // (H // G)
            s = (k[lo:i + 1, g] @ q[i, a]) * scale
            if slopes is not None:
                s = s - slopes[a] * (i - torch.arange(lo, i + 1, dtype=F))
            vals = v[lo:i + 1, g]
            if nvis:
                s = torch.cat([(kb[:nvis, g] @ q[i, a]) * scale, s])
                vals = torch.cat([vb[:nvis, g], vals])
            out[i, a] = torch.softmax(s, dim=0) @ vals
    return out


def gated_attention_mixer(h, m: dict, W, p: str) -> torch.Tensor:
    """Mixer 'attention': no rotation, distance bias, sliding window, sigmoid gate on the heads."""
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = lin(h, W, p + "q").view(T, H, d)
    k = lin(h, W, p + "k").view(T, G, d)
    v = lin(h, W, p + "v").view(T, G, e)
    o = softmax_attention(q, k, v, float(m["scale"]), int((m.get("mask") or {}).get("size") or 0), 0, distance_slopes(H))
    o = o.reshape(T, H * e) * torch.sigmoid(lin(h, W, p + "g"))
    return lin(o, W, p + "o")


def pooled_window_mixer(h, m: dict, W, p: str, eps: float) -> torch.Tensor:
    """Left member of 'parallel': per-head query/key norm, rotation, window with pooled blocks."""
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms_norm(lin(h, W, p + "q").view(T, H, d), W[p + "q.norm"], eps)
    k = rms_norm(lin(h, W, p + "k").view(T, G, d), W[p + "k.norm"], eps)
    q, k = rotate_halves(q, m.get("rot")), rotate_halves(k, m.get("rot"))
    v = lin(h, W, p + "v").view(T, G, e)
    mask = m.get("mask") or {}
    o = softmax_attention(q, k, v, float(m["scale"]), int(mask.get("size") or 0), int(mask.get("pool") or 0))
    return lin(o.reshape(T, H * e), W, p + "o")


# ----------------------------------------------------------------------------- retention
def retention_mixer(h, m: dict, W, p: str, eps: float, state: Optional[torch.Tensor] = None, return_state: bool = False):
    """Right member of 'parallel': S <- decay * S + k v^T, o = S^T q per head, no softmax."""
    T = h.shape[0]
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = rotate_halves(lin(h, W, p + "q").view(T, H, d), m.get("rot"))
    k = rotate_halves(lin(h, W, p + "k").view(T, H, d), m.get("rot")) * d ** -0.5
    v = lin(h, W, p + "v").view(T, H, e)
    decay = torch.tensor([float(x) for x in m["decay"]], dtype=F)
    S = torch.zeros(H, d, e, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, e, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    o = rms_unit(o, eps).reshape(T, H * e) * silu(lin(h, W, p + "g"))
    out = lin(o, W, p + "o")
    return (out, S) if return_state else out


def parallel_mixer(h, m: dict, W, p: str, eps: float) -> torch.Tensor:
    left = pooled_window_mixer(h, m["left"], W, p + "left.", eps)
    right = retention_mixer(h, m["right"], W, p + "right.", eps)
    return 0.5 * (rms_norm(left, W[p + "left.out"], eps) + rms_norm(right, W[p + "right.out"], eps))


# ----------------------------------------------------------------------------- feed-forward
def gated_expert(h, W, p: str) -> torch.Tensor:
    return lin(silu(lin(h, W, p + "gate")) * lin(h, W, p + "up"), W, p + "down")


def route(scores: torch.Tensor, top: int, groups: int, keep: int):
    """scores [E] -> (chosen experts, their weights): the ``top`` largest among the experts of the ``keep`` groups
    (of E / groups neighbours each) whose largest score is largest; weights are the scores over their sum."""
    E = scores.shape[0]
    allowed = torch.ones(E, dtype=torch.bool)
    if groups > 1 and keep < groups:
        best = scores.view(groups, E // groups).max(dim=1).values
        kept = torch.topk(best, keep).indices
        allowed = torch.zeros(groups, E // groups, dtype=torch.bool)
        allowed[kept] = True
        allowed = allowed.view(E)
    masked = torch.where(allowed, scores, torch.full_like(scores, -1.0))
    chosen = torch.topk(masked, top).indices
    w = scores[chosen]
    return chosen, w / (w.sum() + 1e-20)


def moe_feed_forward(h, mlp: dict, W, p: str) -> torch.Tensor:
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    grp = r.get("groups") or {}
    scores = torch.softmax(lin(h, W, p + "router"), dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, w = route(scores[t], top, int(grp.get("count") or 1), int(grp.get("keep") or 1))
        for e_, w_ in zip(chosen.tolist(), w):
            out[t] += w_ * gated_expert(h[t:t + 1], W, f"{p}e{e_}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, W, p + "shared.")
    return out


# ----------------------------------------------------------------------------- the model
def run_layer(x, L: dict, W, p: str, eps: float) -> torch.Tensor:
    h = rms_norm(x, W[p + "norm1"], eps)
    if L["type"] == "attention":
        y = gated_attention_mixer(h, L["mixer"], W, p + "mix.")
    elif L["type"] == "parallel":
        y = parallel_mixer(h, L["mixer"], W, p + "mix.", eps)
    else:
        raise ValueError(L["type"])
    x = x + rms_norm(y, W[p + "norm1b"], eps)
    if L.get("mlp") is not None:
        y = moe_feed_forward(rms_norm(x, W[p + "norm2"], eps), L["mlp"], W, p + "mlp.")
        x = x + rms_norm(y, W[p + "norm2b"], eps)
    return x


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits [T, vocab] (float64) of one sequence.  ``return_layers``: also what every layer hands on, [layers, T, width]."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"].to(F)[torch.tensor(tokens, dtype=torch.long)]
    results = [x]                                   # the embedding output, then every layer's own result
    handed = []
    for i, L in enumerate(cfg["layers"]):
        results.append(run_layer(x, L, W, f"l{i}.", eps))
        a = W[f"l{i}.dwa"].to(F)
        x = sum(a[j] * results[j] for j in range(i + 2))
        handed.append(x)
    logits = lin(rms_norm(x, W["final.norm"], eps), W, "embed")
    return (logits, torch.stack(handed)) if return_layers else logits


def load_model_folder(folder, dtype=F):
    """(config dictionary, name -> tensor) of a folder with config.json and model.safetensors, read with nothing but
    the standard library and torch."""
    import json
    import struct
    from pathlib import Path
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    types = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64, "I32": torch.int32}
    W = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=types[info["dtype"]]).reshape(info["shape"])
        W[name] = t.to(dtype) if t.dtype.is_floating_point else t
    return cfg, W


# ----------------------------------------------------------------------------- random models for the tests
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Name -> shape of every tensor of a model."""
    W = int(cfg["width"])
    out = {"embed": (int(cfg["vocab"]), W), "final.norm": (W,)}

    def softmax_member(p, m, gate):
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "q": (H * d, W), p + "k": (G * d, W), p + "v": (G * e, W), p + "o": (W, H * e)})
        if gate:
            out[p + "g"] = (H * e, W)
        else:
            out.update({p + "q.norm": (d,), p + "k.norm": (d,)})

    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out.update({p + "norm1": (W,), p + "norm1b": (W,), p + "dwa": (i + 2,)})
        if L["type"] == "attention":
            softmax_member(p + "mix.", m, True)
        else:
            softmax_member(p + "mix.left.", m["left"], False)
            r = m["right"]
            H, d, e = r["heads"], r["dim"], r["vdim"]
            q = p + "mix.right."
            out.update({q + "q": (H * d, W), q + "k": (H * d, W), q + "v": (H * e, W), q + "g": (H * e, W), q + "o": (W, H * e),
                        p + "mix.left.out": (W,), p + "mix.right.out": (W,)})
        mlp = L.get("mlp")
        if mlp:
            out.update({p + "norm2": (W,), p + "norm2b": (W,)})
            ff = mlp["expert"]["ff"]
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for x in range(mlp["router"]["experts"]):
                out.update({f"{p}mlp.e{x}.gate": (ff, W), f"{p}mlp.e{x}.up": (ff, W), f"{p}mlp.e{x}.down": (W, ff)})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
    return out


def random_weights(cfg: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Weights drawn so that no mechanism drowns: matrices N(0, 1.5^2 / fan_in), norm weights around one, depth
    coefficients of either sign that give every result a say, router logits that spread.  In 16 bits scores are
    smaller and the depth coefficients positive: a score s carries a rounding error of about |s| * 2^-8, and a
    difference of two results of similar size multiplies every rounding error before it."""
    gentle = dtype != torch.float32
    gen = torch.Generator().manual_seed(seed)
    rand = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
    uni = lambda lo, hi, *s: lo + (hi - lo) * torch.rand(*s, generator=gen, dtype=torch.float32)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        last = name.split(".")[-1]
        if name == "embed":
            t = rand(*shape) * 0.7
        elif last in ("norm1", "norm2", "norm1b", "norm2b", "norm", "out") or name == "final.norm":
            t = 1 + 0.2 * rand(*shape)
        elif last == "dwa":
            t = uni(0.3, 0.9, *shape) * torch.where((torch.arange(shape[0]) % 3 == 1) & (not gentle), -1.0, 1.0)
            t[-1] = t[-1].abs() + 0.3
            if gentle:
                t = t / t.sum()
        elif last == "router":
            t = rand(*shape) * (3.0 / math.sqrt(shape[-1]))
        elif last in ("q", "k"):
            t = rand(*shape) * ((1.2 if gentle else 2.5) / math.sqrt(shape[-1]))
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


def rotation(dims, base):
    return {"dims": dims, "base": base}


def gated_attention(heads, kv_heads, dim, vdim, scale, size=0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    return m


def pooled_attention(heads, kv_heads, dim, vdim, scale, size=0, pool=0, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size, **({"pool": pool} if pool else {})}
    if rot:
        m["rot"] = rot
    return m


def retention(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = rot
    return m


def parallel(left, right):
    return {"left": left, "right": right}


def moe(ff, experts, top, groups=0, keep=0, shared=0):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(vocab, width, layers, eps=1e-5):
    return {"architecture": "Podizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# A parallel layer first; windows and pooled blocks that straddle pages of 4, 8 and 16; value heads larger and smaller
# than key heads; half a head rotated on the left, a whole head on the right; a layer without a feed-forward; groups
# of three experts of which two are kept; a router without groups.
TINY_A = config(97, 48, [
    layer("parallel", parallel(pooled_attention(4, 2, 16, 24, 0.3, size=11, pool=5, rot=rotation(8, 1000.0)),
                               retention(3, 8, 12, (0.9, 0.97, 0.995), rot=rotation(8, 50.0))), moe(24, 6, 2, groups=2, keep=1, shared=16)),
    layer("attention", gated_attention(4, 1, 16, 8, 0.25, size=9), moe(16, 4, 3)),
    layer("parallel", parallel(pooled_attention(2, 2, 24, 16, 0.2, size=6, pool=7, rot=rotation(24, 300.0)),
                               retention(1, 20, 40, (0.98,), rot=rotation(4, 10.0))), None),
    layer("attention", gated_attention(6, 3, 8, 8, 0.4, size=17), moe(12, 9, 3, groups=3, keep=2)),
])
# An attention layer first; as many kv heads as heads; every group kept and every expert chosen; a window of one block;
# blocks of one position; a retention that forgets at once and one that never does; no rotation on the right.
TINY_B = config(70, 64, [
    layer("attention", gated_attention(6, 6, 16, 16, 0.35, size=7), moe(24, 3, 3, groups=3, keep=3, shared=24)),
    layer("parallel", parallel(pooled_attention(3, 1, 16, 32, 0.3, size=4, pool=4, rot=rotation(16, 50.0)),
                               retention(2, 32, 8, (0.0, 1.0))), moe(16, 8, 2, groups=4, keep=2)),
    layer("parallel", parallel(pooled_attention(2, 1, 32, 8, 0.2, size=9, pool=1),
                               retention(2, 12, 20, (0.5, 0.999), rot=rotation(12, 1.0e6))), None),
], eps=3e-4)
# A window without pooled blocks, an attention that sees everything, one expert of one, a width that is no multiple of
# eight.
TINY_C = config(50, 36, [
    layer("parallel", parallel(pooled_attention(3, 1, 16, 32, 0.3, size=8, rot=rotation(16, 50.0)),
                               retention(2, 8, 8, (0.9, 0.8), rot=rotation(8, 7.0))), moe(16, 1, 1, shared=8)),
    layer("attention", gated_attention(3, 1, 16, 32, 0.3), moe(8, 6, 1, groups=6, keep=1)),
    layer("parallel", parallel(pooled_attention(1, 1, 8, 8, 0.5, rot=rotation(2, 3.0)),
                               retention(1, 8, 16, (0.95,))), None),
])
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
