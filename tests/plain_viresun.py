"""A plain, slow implementation of the Viresun decoder for the tests: one function per mechanism,
whole sequences, torch on the CPU in the precision the caller chooses (float64 by default).
It shares nothing with the engine: it reads a configuration dictionary and tensors by name.

Notation: ``T`` tokens, ``W`` the width of the residual stream, positions ``0 .. T-1``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# ---- small pieces ------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """Every last-dimension vector divided by sqrt(mean of its squares + eps)."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is one number."""
    return unit_rms(x, eps) * g


def sinusoid_rows(T: int, W: int, dtype) -> torch.Tensor:
    """Row p: sin(p / 10000^(2i/W)) at column 2i, the cosine of the same angle at 2i+1."""
    out = torch.zeros(T, W, dtype=dtype)
    for i in range(W // 2):
        angle = torch.arange(T, dtype=dtype) * (10000.0 ** (-2.0 * i / W))
        out[:, 2 * i] = torch.sin(angle)
        out[:, 2 * i + 1] = torch.cos(angle)
    return out


def embed(tokens: Sequence[int], table: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    x = table[torch.tensor(list(tokens))]
    return scalar_norm(x + sinusoid_rows(len(tokens), table.shape[1], x.dtype), g, eps)


# ---- attention -----------------------------------------------------------------------------
def query_temperature(T: int, coef: float, every: int, dtype) -> torch.Tensor:
    p = torch.arange(T)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(dtype))


def biased_window_attention(q, k, v, scale: float, window: Optional[int], r1, r2) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, E] -> [T, H, E]; one query row at a time."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        lo = 0 if not window else max(0, i - window + 1)
        dist = torch.arange(i - lo, -1, -1, dtype=q.dtype)            # i - j for j = lo .. i
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            if r1 is not None:
                s = s - r1[h] * torch.log(1.0 + r2[h] * dist)
            out[i, h] = torch.softmax(s, dim=0) @ v[lo:i + 1, g]
    return out


def attention_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ w[p + "q"].T).view(T, H, D), eps)
    k = unit_rms((h @ w[p + "k"].T).view(T, G, D), eps)
    v = (h @ w[p + "v"].T).view(T, G, E)
    if m.get("q_temp"):
        q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype)[:, None, None]
    window = (m.get("mask") or {}).get("size")
    o = biased_window_attention(q, k, v, m["scale"], window, w[p + "r1"], w[p + "r2"])
    return o.reshape(T, H * E) @ w[p + "o"].T


# ---- Mamba-2 -------------------------------------------------------------------------------
def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(u: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """u [T, C]; weight [C, taps]: tap j weighs the row taps-1-j tokens back; rows of negative index are zero."""
    T, C = u.shape
    taps = weight.shape[1]
    out = bias.expand(T, C).clone()
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += weight[:, j] * u[src]
    return out


def ssm_recurrence(x, B, C, dt, a_log, d_skip) -> torch.Tensor:
    """x [T, Hh, E], B and C [T, G, N], dt [T, Hh] (after softplus) -> y [T, Hh, E]."""
    T, Hh, E = x.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(x)
    for h in range(Hh):
        g = h // (Hh // G)
        S = torch.zeros(N, E, dtype=x.dtype)
        rate = torch.exp(a_log[h])
        for t in range(T):
            S = torch.exp(-rate * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + d_skip[h] * x[t, h]
    return y


def mamba2_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    Hh, E, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hh * E
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, Hh, E)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.log1p(torch.exp(dt + w[p + "dt_bias"]))
    y = ssm_recurrence(x, B, C, dt, w[p + "A_log"], w[p + "D"]).reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# ---- feed-forwards -------------------------------------------------------------------------
def dense_feed_forward(h, w, p: str) -> torch.Tensor:
    return (torch.relu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert(hrow, w, p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(w[p + "gate"] @ hrow, max=limit)
    u = torch.clamp(w[p + "up"] @ hrow, -limit, limit)
    return w[p + "down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def route(h, w, p: str, top: int):
    """(chosen [T, top], weights [T, top]) by the largest router logits."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    best, chosen = torch.topk(z, top, dim=1)
    return chosen, torch.softmax(best, dim=1)


def routed_feed_forward(h, w, p: str, mlp: dict) -> torch.Tensor:
    chosen, share = route(h, w, p, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c, e in enumerate(chosen[t].tolist()):
            out[t] += share[t, c] * expert(h[t], w, f"{p}e{e}.", mlp["expert"]["limit"])
    return out


# ---- the whole model -------------------------------------------------------------------------
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64,
            residuals: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = embed(tokens, w["embed"], w["embed.norm"], eps)
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        h = scalar_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            x = x + attention_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            x = x + mamba2_mixer(h, w, p + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = scalar_norm(x, w[p + "norm2"], eps)
            x = x + (dense_feed_forward(h, w, p + "mlp.") if mlp["kind"] == "dense"
                     else routed_feed_forward(h, w, p + "mlp.", mlp))
        if residuals is not None:
            residuals.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(config: dict, weights, prompt: Sequence[int], n: int, dtype=torch.float64) -> List[int]:
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(config, weights, tokens, dtype)[-1].argmax()))
    return tokens[len(prompt):]


# ---- tensors of a configuration, drawn so that every mechanism matters ------------------------
def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V = config["width"], config["vocab"]
    out = {"embed": (V, W), "embed.norm": (), "final.norm": (), "head": (V, W)}
    for i, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = ()
        if layer["type"] == "attention":
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * D, W), p + "mix.k": (G * D, W), p + "mix.v": (G * E, W),
                        p + "mix.o": (W, H * E), p + "mix.r1": (H,), p + "mix.r2": (H,)})
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out.update({p + "mix.in": (2 * inner + 2 * gn + m["heads"], W), p + "mix.conv": (inner + 2 * gn, m["conv"]),
                        p + "mix.conv.b": (inner + 2 * gn,), p + "mix.dt_bias": (m["heads"],),
                        p + "mix.A_log": (m["heads"],), p + "mix.D": (m["heads"],), p + "mix.norm": (inner,),
                        p + "mix.o": (W, inner)})
        mlp = layer.get("mlp")
        if mlp:
            out[p + "norm2"] = ()
            if mlp["kind"] == "dense":
                out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
                out.update({p + "mlp.router": (E, W), p + "mlp.router.b": (E,)})
                for e in range(E):
                    out.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
    return out


def random_tensors(config: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Tensors in float32 whose values are exact in bfloat16.  Matrices have rows of unit length on
    average, so that every stage's output is of the order of one: no mechanism drowns, and none
    multiplies the rounding of the stage before it."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if shape == ():
            t = 1.0 + 0.2 * torch.rand((), generator=g)
        elif leaf == "r1":
            t = 0.5 + torch.rand(shape, generator=g)
        elif leaf == "r2":
            t = 0.05 + 0.5 * torch.rand(shape, generator=g)
        elif leaf == "A_log":
            t = torch.log(0.02 + 0.3 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g) - 0.5
        elif leaf == "D":
            t = torch.randn(shape, generator=g)
        elif name.endswith("conv"):
            t = torch.randn(shape, generator=g) * 0.6
        elif name.endswith("mix.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
