"""Small Viresun configurations for the tests.  Between them every size differs, sizes that are
often equal are not (key and value size, heads and key/value heads, groups and heads), values
that are often 1 are not, and the branches a configuration may leave out are left out once."""


def attention(heads, kv_heads, dim, vdim, scale, window=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


# key size 24, value size 40, 6 heads on 2; window 21 (not a multiple of a page, longer than one);
# temperature steps every 16 positions; Mamba with 3 groups of 2 heads, 4 taps, 3 norm groups;
# 6 experts, 2 chosen; a layer without a feed-forward; layer 4 runs layer 1's tensors
VIRESUN_A = {
    "architecture": "Viresun", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": attention(6, 2, 24, 40, 0.21, window=21, q_temp=(0.4, 16)), "mlp": dense(88)},
        {"type": "mamba2", "mixer": mamba(6, 12, 20, 3, 4, 3), "mlp": moe(40, 6, 2, 1.25)},
        {"type": "attention", "mixer": attention(6, 2, 24, 40, 0.21, window=21, q_temp=(0.4, 16)), "mlp": None},
        {"type": "attention", "mixer": attention(4, 4, 16, 16, 0.3, window=5), "mlp": moe(24, 5, 1, 2.0)},
        {"type": "mamba2", "mixer": mamba(6, 12, 20, 3, 4, 3), "mlp": moe(40, 6, 2, 1.25), "weights_of": 1},
    ],
}
# widths that are multiples of 8 (the tensor-core products run in bfloat16), head size 64 and 32,
# one key/value head, a window longer than the prompts (never cuts), no temperature in one layer and no
# window in another; Mamba with one group, 2 taps, one norm group, a state of 70 (more than 64);
# 9 experts, 3 chosen
VIRESUN_B = {
    "architecture": "Viresun", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mamba2", "mixer": mamba(4, 32, 70, 1, 2, 1), "mlp": dense(192)},
        {"type": "attention", "mixer": attention(4, 1, 64, 32, 0.125, window=400), "mlp": moe(64, 9, 3, 1.5)},
        {"type": "attention", "mixer": attention(2, 2, 32, 64, 0.2, q_temp=(0.25, 7)), "mlp": dense(64)},
    ],
}
# a width that is no multiple of 8 (no tensor-core product takes it), head sizes 20 and 12, a window of one (a row
# sees itself alone) beside none, a convolution of one tap (no inputs carried), every Mamba head its own group and
# norm part, an attention layer that borrows tensors, 3 experts of which 2 are chosen, an odd vocabulary
VIRESUN_C = {
    "architecture": "Viresun", "vocab": 97, "width": 44, "norm": {"eps": 3e-6},
    "layers": [
        {"type": "attention", "mixer": attention(3, 3, 20, 12, 0.4, window=1, q_temp=(1.0, 3)), "mlp": moe(16, 3, 2, 0.8)},
        {"type": "mamba2", "mixer": mamba(2, 10, 6, 2, 1, 2), "mlp": None},
        {"type": "attention", "mixer": attention(4, 2, 12, 20, 0.35), "mlp": dense(52)},
        {"type": "attention", "mixer": attention(3, 3, 20, 12, 0.4, window=1, q_temp=(1.0, 3)), "mlp": moe(16, 3, 2, 0.8),
         "weights_of": 0},
    ],
}
# no attention at all (no page group, states only), and no recurrent mixer at all (pages only)
VIRESUN_ONLY_MAMBA = {
    "architecture": "Viresun", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
    "layers": [{"type": "mamba2", "mixer": mamba(2, 8, 12, 1, 3, 2), "mlp": dense(40)},
               {"type": "mamba2", "mixer": mamba(4, 4, 5, 2, 2, 1), "mlp": moe(16, 4, 2, 1.0)}],
}
VIRESUN_ONLY_ATTENTION = {
    "architecture": "Viresun", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
    "layers": [{"type": "attention", "mixer": attention(2, 1, 16, 8, 0.25, window=9), "mlp": None},
               {"type": "attention", "mixer": attention(4, 4, 8, 8, 0.3, q_temp=(0.5, 4)), "mlp": dense(48)}],
}
CONFIGS = {"A": VIRESUN_A, "B": VIRESUN_B, "C": VIRESUN_C}
