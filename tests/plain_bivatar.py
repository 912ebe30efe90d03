"""A plain, slow implementation of the Bivatar decoder for the tests: one function per mechanism,
whole sequences, torch on the CPU in the precision the caller chooses (float64 by default).
It shares nothing with the engine: it reads a configuration dictionary and tensors by name.

Notation: ``T`` tokens at positions ``0 .. T-1``, ``W`` the width of the residual stream, ``H`` query
heads.  A weight ``[out, in]`` acts as ``h @ weight.T``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# ---- small pieces ------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Every last-dimension vector divided by sqrt(mean of its squares + eps), times the weight."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_feed_forward(h, gate, up, down) -> torch.Tensor:
    return (gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


# ---- rotation with stretched frequencies ---------------------------------------------------
def stretched_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency of every pair ``[dims/2]``, factor on cosine and sine).

    Pair ``i`` turns by ``base^(-2i/dims)`` per position.  With ``scaling`` (factor ``s``, trained
    length ``n``, turn counts ``fast`` and ``slow``): the pair that makes ``t`` turns over ``n``
    positions has the (real-valued) index ``d(t) = dims ln(n / (2 pi t)) / (2 ln base)``; pairs below
    ``floor(d(fast))`` keep their frequency, pairs above ``ceil(d(slow))`` have it divided by ``s``,
    and in between the two are blended linearly in ``i``.  Cosine and sine grow by ``0.1 ln s + 1``."""
    half = dims // 2
    freq = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return freq, 1.0
    s, n = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(n / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(freq[i] / s * ramp + freq[i] * (1.0 - ramp))
    return out, 0.1 * math.log(s) + 1.0


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, freq: Sequence[float], grow: float) -> torch.Tensor:
    """v [T, ..., dims]: entry i is paired with entry i + dims/2; the pair at position p turns by p * freq[i]."""
    half = len(freq)
    angle = positions.to(v.dtype)[:, None] * torch.tensor(freq, dtype=v.dtype)[None, :]      # [T, half]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = (torch.cos(angle) * grow).view(shape), (torch.sin(angle) * grow).view(shape)
    a, b = v[..., :half], v[..., half:2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., 2 * half:]], dim=-1)


# ---- attention through a shared latent -----------------------------------------------------
def latent_keys(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """What a layer with a down-projection of its own keeps per token: the normed latent ``[T, R]`` and
    the rotated key part ``[T, rot]`` that all heads share."""
    T, R, rot = h.shape[0], m["kv_rank"], m["rot_dim"]
    down = h @ w[p + "dkv"].T
    latent = rms_norm(down[:, :R], w[p + "dkv.norm"], eps)
    freq, grow = stretched_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    shared = rotate_pairs(down[:, R:R + rot], torch.arange(T), freq, grow)
    return latent, shared


def latent_attention(q, q_rot, latent, shared, uk, uv, scale: float) -> torch.Tensor:
    """q [T, H, D] unrotated and q_rot [T, H, rot] rotated query parts, latent [S, R] and shared [S, rot]
    of the S >= T tokens so far (the queries are the last T), uk [H*D, R], uv [H*E, R] -> [T, H, E].
    Keys and values are formed per head, as the design writes them."""
    T, H, D = q.shape
    S = latent.shape[0]
    E = uv.shape[0] // H
    k = (latent @ uk.T).view(S, H, D)
    v = (latent @ uv.T).view(S, H, E)
    out = torch.zeros(T, H, E, dtype=q.dtype)
    for t in range(T):
        i = S - T + t
        for a in range(H):
            s = (k[:i + 1, a] @ q[t, a] + shared[:i + 1] @ q_rot[t, a]) * scale
            out[t, a] = torch.softmax(s, dim=0) @ v[:i + 1, a]
    return out


def latent_attention_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, kept) -> torch.Tensor:
    """``kept``: (latent, shared rotated key part) of this layer or of the layer it reads them from."""
    T = h.shape[0]
    H, D, rot, E = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    latent, shared = kept
    q = (rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps) @ w[p + "uq"].T).view(T, H, D + rot)
    freq, grow = stretched_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q_rot = rotate_pairs(q[..., D:], torch.arange(T), freq, grow)
    out = latent_attention(q[..., :D], q_rot, latent, shared, w[p + "uk"], w[p + "uv"], m["scale"])
    out = out * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return out.reshape(T, H * E) @ w[p + "o"].T


# ---- windowed attention with a linear distance penalty -------------------------------------
def head_slopes(H: int) -> List[float]:
    return [2.0 ** (-8.0 * (a + 1) / H) for a in range(H)]


def visible(i: int, j: int, window: Optional[int], keep_first: int) -> bool:
    return j <= i and (window is None or i - j < window or j < keep_first)


def sloped_window_attention(q, k, v, scale: float, window: Optional[int], keep_first: int) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, E] -> [T, H, E]; one query row at a time over the keys it sees."""
    T, H, _ = q.shape
    G = k.shape[1]
    slopes = head_slopes(H)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
        idx = torch.tensor(js)
        dist = torch.tensor([float(i - j) for j in js], dtype=q.dtype)
        for a in range(H):
            g = a // (H // G)
            s = (k[idx, g] @ q[i, a]) * scale - slopes[a] * dist
            out[i, a] = torch.softmax(s, dim=0) @ v[idx, g]
    return out


def window_attention_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    mask = m.get("mask") or {}
    q = rms_norm((h @ w[p + "q"].T).view(T, H, D), w[p + "q.norm"], eps)
    k = rms_norm((h @ w[p + "k"].T).view(T, G, D), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).view(T, G, E)
    out = sloped_window_attention(q, k, v, m["scale"], mask.get("size"), int(mask.get("keep_first") or 0))
    out = out * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return out.reshape(T, H * E) @ w[p + "o"].T


# ---- the whole model -----------------------------------------------------------------------
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence; ``layers_out`` collects the residual stream after every layer."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    x = w["embed"][torch.tensor(list(tokens))] * float(config["embedding"]["scale"])
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_keys(x, w, p, m, eps)
                src = i
            y = latent_attention_mixer(x, w, p, m, eps, kept[src])
        elif layer["type"] == "attention":
            y = window_attention_mixer(x, w, p, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * rms_norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp"):
            y = gated_feed_forward(x, w[f"l{i}.mlp.gate"], w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"])
            x = x + mult * rms_norm(y, w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


# ---- tensors of a configuration ------------------------------------------------------------
def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V = config["width"], config["vocab"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (W,)
        if layer["type"] == "latent_attention":
            H, D, rot, E, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({p + "mix.dq": (Q, W), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (D + rot), Q),
                        p + "mix.uk": (H * D, R), p + "mix.uv": (H * E, R), p + "mix.g": (H, W),
                        p + "mix.o": (W, H * E)})
            if m.get("kv_from") is None:
                out.update({p + "mix.dkv": (R + rot, W), p + "mix.dkv.norm": (R,)})
        else:
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * D, W), p + "mix.k": (G * D, W), p + "mix.v": (G * E, W),
                        p + "mix.q.norm": (D,), p + "mix.k.norm": (D,), p + "mix.g": (H, W), p + "mix.o": (W, H * E)})
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            out.update({p + "norm2": (W,), p + "mlp.gate": (F, W), p + "mlp.up": (F, W), p + "mlp.down": (W, F)})
    return out


def random_tensors(config: dict, seed: int, spread: float = 2.0) -> Dict[str, torch.Tensor]:
    """Random tensors (float64, every value a bfloat16 number): matrices with a spread of
    ``spread / sqrt(in)``, norm weights around one.  With a spread of 2 scores and gates move far and the
    softmax is sharp, which shows a wrong key at once but also carries rounding a long way; the bfloat16
    tests take a spread of 1."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        if len(shape) == 1:
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen, dtype=torch.float64)
        elif name == "embed":
            t = torch.randn(shape, generator=gen, dtype=torch.float64)
        else:
            t = torch.randn(shape, generator=gen, dtype=torch.float64) * (spread / math.sqrt(shape[1]))
        out[name] = t.to(torch.bfloat16).to(torch.float64)
    return out


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int], n: int) -> List[int]:
    """``n`` tokens chosen by the largest logit, the whole sequence recomputed for each."""
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(forward(config, weights, toks)[-1]))
        out.append(t)
        toks.append(t)
    return out
