"""Small Bivatar configurations for the tests.  Between them every size differs, sizes that are
often equal are not (unrotated and rotated dimensions, value size and latent, heads and key/value
heads, the sizes of layers that share a latent), constants that are often 1 or equal are not
(the residual factor, the embedding scale), and the branches a configuration may leave out are
left out once (frequency scaling, window, kept first tokens, feed-forward)."""


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rotation, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale, "rot": rotation}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def window(heads, kv_heads, dim, vdim, scale, size=None, keep_first=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


ROT_A = rot(16, 10000.0, (4.0, 64, 8.0, 1.0))      # stretched: the ramp covers pairs 2 to 6 of 8
ROT_A2 = rot(8, 500.0)                             # plain frequencies
# 3 heads of 24 + 16, values of 40, latent 48, query latent 56; window 21 with 5 kept first tokens (neither a
# multiple of a page); layer 2 reads layer 0's latent with 5 heads of other sizes and has no feed-forward;
# layer 3 keeps a latent of another width; layer 5 reads layer 3's; one key/value head per query head in layer 4
BIVATAR_A = {
    "architecture": "Bivatar", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.8,
    "embedding": {"scale": 1.5},
    "layers": [
        layer("latent_attention", latent(3, 24, 16, 40, 48, 56, 0.17, ROT_A), dense(88)),
        layer("attention", window(6, 2, 24, 40, 0.21, size=21, keep_first=5), dense(72)),
        layer("latent_attention", latent(5, 8, 16, 16, 48, 24, 0.3, ROT_A, kv_from=0), None),
        layer("latent_attention", latent(2, 32, 8, 24, 40, 32, 0.15, ROT_A2), dense(64)),
        layer("attention", window(4, 4, 16, 16, 0.3, size=5), dense(48)),
        layer("latent_attention", latent(4, 16, 8, 8, 40, 16, 0.25, ROT_A2, kv_from=3), dense(40)),
    ],
}
# a residual factor and an embedding scale of one; an attention layer without a window, one whose window never
# cuts (but keeps first tokens) on a single key/value head, a window shorter than the kept first tokens;
# a rotation that turns only 8 of the 16 rotated dimensions, 9 heads (more than 8 share the one latent)
BIVATAR_B = {
    "architecture": "Bivatar", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
    "embedding": {"scale": 1.0},
    "layers": [
        layer("attention", window(4, 1, 64, 32, 0.125, size=400, keep_first=3), dense(192)),
        layer("latent_attention", latent(9, 16, 16, 24, 80, 64, 0.2, rot(8, 1000.0, (16.0, 32, 4.0, 0.5))), dense(64)),
        layer("attention", window(2, 2, 32, 64, 0.2), None),
        layer("attention", window(8, 4, 16, 24, 0.3, size=6, keep_first=19), dense(96)),
    ],
}
# a width that is no multiple of 8 (no tensor-core product takes it), head sizes 20 and 12, a window of one beside
# two kept tokens, a latent of 20 with 6 rotated dimensions, a single head, an odd vocabulary, sharing across an
# attention layer
BIVATAR_C = {
    "architecture": "Bivatar", "vocab": 97, "width": 44, "norm": {"eps": 3e-6}, "residual_mult": 0.35,
    "embedding": {"scale": 0.7},
    "layers": [
        layer("latent_attention", latent(1, 12, 6, 20, 20, 28, 0.4, rot(6, 50.0, (2.0, 16, 2.0, 0.25))), dense(52)),
        layer("attention", window(3, 3, 20, 12, 0.4, size=1, keep_first=2), None),
        layer("latent_attention", latent(2, 10, 6, 14, 20, 12, 0.35, rot(6, 50.0, (2.0, 16, 2.0, 0.25)), kv_from=0),
              dense(36)),
    ],
}
ONLY_LATENT = {
    "architecture": "Bivatar", "vocab": 64, "width": 32, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
    "embedding": {"scale": 2.0},
    "layers": [layer("latent_attention", latent(2, 8, 8, 8, 16, 16, 0.3, rot(8, 100.0)), dense(40)),
               layer("latent_attention", latent(4, 4, 8, 12, 16, 8, 0.3, rot(8, 100.0), kv_from=0), dense(24))],
}
ONLY_WINDOW = {
    "architecture": "Bivatar", "vocab": 64, "width": 32, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
    "embedding": {"scale": 2.0},
    "layers": [layer("attention", window(2, 1, 16, 8, 0.25, size=9, keep_first=4), None),
               layer("attention", window(4, 4, 8, 8, 0.3), dense(48))],
}
# a latent wider than the tensor-core attention kernel takes (136 + 16): prompt portions in bfloat16 run on keys
# and values formed per head, single rows in the latent space; a second layer reads the same latent
BIVATAR_D = {
    "architecture": "Bivatar", "vocab": 128, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
    "embedding": {"scale": 1.2},
    "layers": [
        layer("latent_attention", latent(3, 24, 16, 40, 136, 32, 0.17, ROT_A), dense(64)),
        layer("attention", window(2, 1, 16, 24, 0.25, size=30, keep_first=9), None),
        layer("latent_attention", latent(5, 40, 16, 8, 136, 48, 0.14, ROT_A, kv_from=0), dense(40)),
    ],
}
CONFIGS = {"A": BIVATAR_A, "B": BIVATAR_B, "C": BIVATAR_C, "D": BIVATAR_D}
