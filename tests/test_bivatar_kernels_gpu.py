"""Each mechanism of the Bivatar decoder alone, kernel against the plain implementation, with
inputs made so that a fault shows: one key whose score stands out, far away among hundreds, just
inside and just outside the window, the last kept first token and the first that is not kept, at
page borders, in prompt portions and in single decoded rows; pages that were given back are filled
with NaN."""
import math

import pytest
import torch

import plain_bivatar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def close(got, want, tol, what):
    got, want = got.double().cpu(), want.double()
    err = float((got - want).abs().max() / want.abs().max().clamp(min=1e-30))
    assert torch.isfinite(got).all() and err <= tol, (what, err)


def paged(rows, P, order):
    """rows [T, G, F] of one sequence -> pages [n, G, P, F] with the sequence's pages at the places
    ``order`` names, NaN where nothing was written but zero behind the last token of a page."""
    T, G, F = rows.shape
    n = -(-T // P)
    pages = torch.full((max(order) + 1, G, P, F), float("nan"))
    for b in range(n):
        part = rows[b * P:(b + 1) * P]
        pages[order[b], :, :part.shape[0]] = part.transpose(0, 1)
        pages[order[b], :, part.shape[0]:] = 0.0
    return pages, order[:n]


def shuffled(n, base):
    return [base + (7 * b + 3) % n for b in range(n)] if math.gcd(7, n) == 1 else [base + n - 1 - b for b in range(n)]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,G,D,E,P,window,keep", [
    (6, 2, 24, 40, 8, 21, 5), (4, 2, 64, 48, 16, 70, 18), (3, 1, 16, 80, 16, None, 0), (8, 8, 128, 32, 32, 300, 33),
    (2, 2, 32, 32, 8, 1, 2), (2, 1, 20, 12, 8, 11, 16), (12, 1, 16, 16, 8, 64, 1), (2, 1, 160, 136, 16, 100, 7),
    (4, 4, 48, 24, 16, 40, 64)])
def test_window_attention_with_a_key_that_stands_out(dtype, tol, H, G, D, E, P, window, keep):
    """Two sequences in one launch: a portion of 37 rows behind 300 cached tokens and a single decoded
    row at position 333 of another.  One key is made to dominate for chosen rows: the oldest key the
    window still shows and the one behind it, the last kept first token and the next, a page's first
    and last slot, and (without a window) a key hundreds of tokens back."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + D)
    lens = [(300, 37), (333, 1)]                       # (cached before, rows now)
    scale = 1.0 / math.sqrt(D)
    qs, pages_all, table, want, gates = [], [], [], [], []
    base = 0
    for s, (before, now) in enumerate(lens):
        T = before + now
        q = torch.randn(T, H, D, generator=g)
        k = torch.randn(T, G, D, generator=g)
        v = torch.randn(T, G, E, generator=g)
        gate = 2.0 * torch.randn(T, H, generator=g)
        w = window or T
        spikes = {T - 1: T - w, T - 2: T - 2 - w, before: max(0, before - w + 1), before + 1: (before // P) * P,
                  before + 2: keep - 1, before + 3: keep, T - 4: 17 if not window else T - 4,
                  T - 3: ((T - 3 - min(w, T) + 1 + P - 1) // P) * P + P - 1 if w > 2 * P else T - 3}
        for row, key in spikes.items():
            if 0 <= key <= row < T and row >= before:
                # row `row` looks hard at key `key` (if it sees it): strong enough to beat the distance penalty
                k[key] = 0.3 * k[key] + 12.0 * q[row, ::H // G] / q[row, ::H // G].norm(dim=-1, keepdim=True) * math.sqrt(D)
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
        full = plain.sloped_window_attention(q.double(), k.double(), v.double(), scale, window, keep)
        want.append((full * torch.sigmoid(gate.double())[:, :, None])[before:])
        qs.append(q[before:])
        gates.append(gate[before:])
        n = -(-T // P)
        pg, row = paged(torch.cat([k, v], dim=-1), P, shuffled(n, base))
        pages_all.append(pg[base:])
        table.append(row)
        base += n
    pages = torch.cat(pages_all).to(dtype).to(DEV)
    width = max(len(r) for r in table)
    if window:
        # pages the window has passed were given back (but those of kept first tokens): their table
        # entries are void, their contents gone
        for s, (before, now) in enumerate(lens):
            for b in range(-(-keep // P), (before - window + 1) // P if before - window + 1 > 0 else 0):
                pages[table[s][b]] = float("nan")
                table[s][b] = -1
    bt = i32([r + [-1] * (width - len(r)) for r in table])
    q = torch.cat(qs).reshape(-1, H * D).to(dtype).to(DEV).contiguous()
    # the gate as a strided view of a wider matrix, as the stacked projection hands it over
    wide = torch.zeros(q.shape[0], 5 + H, device=DEV)
    wide[:, 5:] = torch.cat(gates).to(DEV)
    slopes = torch.tensor(plain.head_slopes(H), dtype=torch.float32, device=DEV)
    positions = i32([p for before, now in lens for p in range(before, before + now)])
    for single in (False, True):                       # one kernel for all rows; the decode kernel for the single row
        out = torch.empty(q.shape[0], H * E, dtype=dtype, device=DEV)
        ops.attention_window_bias(q, out, pages, bt, i32([0, 37, 38]), positions, 2, H, G, D, E, scale, window or 0,
                                  slopes, None, single_rows=single, other_rows=True, bias="linear", keep_first=keep,
                                  gate=wide[:, 5:])
        close(out.float().reshape(-1, H, E), torch.cat(want), tol, ("window attention", single))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 2.5e-2)])
@pytest.mark.parametrize("H,D,rot,dims,E,R,P", [(3, 24, 16, 16, 40, 48, 8), (9, 16, 16, 8, 24, 80, 16), (1, 12, 6, 6, 20, 20, 8),
                                                (2, 32, 64, 64, 128, 192, 16), (4, 16, 32, 32, 24, 288, 32),
                                                (16, 8, 8, 8, 8, 24, 16)])
def test_latent_attention_in_the_latent_space(dtype, tol, H, D, rot, dims, E, R, P):
    """Queries carried into the latent space, attention over the pages with the value as the head of
    the key's record, results carried out: against keys and values formed per head.  A portion of 21
    rows behind 400 cached tokens beside a single row at position 260; chosen rows look hard at a key
    hundreds of tokens back, at position 0, and at a page's last slot."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(H * 10 + R)
    lens = [(400, 21), (260, 1)]
    scale = 0.9 / math.sqrt(D + rot)
    freq, grow = plain.stretched_frequencies(dims, 300.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0})
    uk = (torch.randn(H * D, R, generator=g) / math.sqrt(R)).to(torch.bfloat16).double()
    uv = (torch.randn(H * E, R, generator=g) / math.sqrt(R)).to(torch.bfloat16).double()
    qs, pages_all, table, want, gates, pos = [], [], [], [], [], []
    base = 0
    for before, now in lens:
        T = before + now
        q = torch.randn(T, H, D + rot, generator=g).double()
        latent = torch.randn(T, R, generator=g).double()
        shared_raw = torch.randn(T, rot, generator=g).double()
        gate = 2.0 * torch.randn(T, H, generator=g)
        for row, key in {T - 1: 3, before: 0, before + 1: (before // P) * P - 1, T - 2: before - 250}.items():
            if 0 <= key <= row < T and row >= before:
                # every head's unrotated key of token `key` points along that head's query of `row`
                dirs = torch.linalg.lstsq(uk, (q[row, :, :D] / q[row, :, :D].norm(dim=-1, keepdim=True)).reshape(-1, 1)).solution[:, 0]
                latent[key] = 0.2 * latent[key] + 6.0 * math.sqrt(D + rot) * dirs / (uk @ dirs).view(H, D).norm(dim=-1).mean()
        shared = plain.rotate_pairs(shared_raw, torch.arange(T), freq, grow)
        latent, shared = (t.to(dtype).double() for t in (latent, shared))
        q = q.float().double()
        q_rot = plain.rotate_pairs(q[..., D:], torch.arange(T), freq, grow)
        full = plain.latent_attention(q[before:, :, :D], q_rot[before:], latent, shared, uk, uv, scale)
        want.append(full * torch.sigmoid(gate.double())[before:, :, None])
        qs.append(q[before:])
        gates.append(gate[before:])
        pos += list(range(before, T))
        n = -(-T // P)
        pg, row = paged(torch.cat([latent, shared], dim=-1)[:, None, :], P, shuffled(n, base))
        pages_all.append(pg[base:, 0])
        table.append(row)
        base += n
    pages = torch.cat(pages_all).to(dtype).to(DEV)                  # [pages, P, R + rot]
    width = max(len(r) for r in table)
    bt = i32([r + [-1] * (width - len(r)) for r in table])
    rows = len(pos)
    q = torch.cat(qs).reshape(rows, H * (D + rot)).float().to(DEV).contiguous()
    positions = i32(pos)
    inv_freq = torch.tensor(freq, dtype=torch.float64).float().to(DEV)
    cos_sin = torch.empty(rows, dims // 2, 2, device=DEV)
    ops.rope_table(positions, inv_freq, cos_sin, grow)
    wdt = dtype
    uk_dev = uk.view(H, D, R).to(wdt).to(DEV).contiguous()
    uv_dev = uv.view(H, E, R).transpose(1, 2).to(wdt).to(DEV).contiguous()
    qa = torch.empty(rows, H * (R + rot), dtype=dtype, device=DEV)
    ops.head_project(q, uk_dev, qa, H, tail=rot, tail_dims=dims, cos_sin=cos_sin)
    gate = torch.cat(gates).to(DEV).contiguous()
    for single in (False, True):
        ol = torch.empty(rows, H * R, dtype=dtype, device=DEV)
        ops.attention_window_bias(qa, ol, pages, bt, i32([0, 21, 22]), positions, 2, H, 1, R + rot, R, scale, 0,
                                  None, None, single_rows=single, other_rows=True, bias=None, gate=gate,
                                  record=R + rot, value_offset=0)
        out = torch.empty(rows, H * E, dtype=dtype, device=DEV)
        ops.head_project(ol, uv_dev, out, H)
        close(out.float().reshape(rows, H, E), torch.cat(want), tol, ("latent attention", single))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Q,R,rot,dims", [(56, 48, 16, 16), (24, 80, 16, 8), (1536, 512, 64, 64), (28, 20, 6, 6)])
def test_latents_normed_rotated_and_stored(dtype, Q, R, rot, dims):
    from allpaca_b200 import ops
    P, eps, H = 8, 1e-5, 3
    g = torch.Generator().manual_seed(Q)
    positions = [0, 1, 7, 8, 15, 16, 1000, 4097, 23]
    T = len(positions)
    proj = 3.0 * torch.randn(T, 2 + Q + R + rot + H, generator=g)        # two unrelated columns in front, the gate behind
    qw = 1.0 + 0.3 * torch.randn(Q, generator=g)
    kvw = 1.0 + 0.3 * torch.randn(R, generator=g)
    freq, grow = plain.stretched_frequencies(dims, 10000.0, {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 2.0})
    npages = 4097 // P + 1
    pages = torch.zeros(npages, P, R + rot, dtype=dtype, device=DEV)
    bt = i32([[(5 * b + 1) % npages for b in range(npages)]])
    pos = i32(positions)
    cos_sin = torch.empty(T, dims // 2, 2, device=DEV)
    ops.rope_table(pos, torch.tensor(freq, dtype=torch.float64).float().to(DEV), cos_sin, grow)
    cq = torch.empty(T, Q, dtype=dtype, device=DEV)
    ops.latent_prepare(proj.to(DEV), 2, Q, qw.to(DEV), cq, 2 + Q, R, rot, dims, kvw.to(DEV), pages, pos, i32([0] * T), bt,
                       cos_sin, eps)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    close(cq.float(), plain.rms_norm(proj[:, 2:2 + Q].double(), qw.double(), eps), tol, "query latent")
    latent = plain.rms_norm(proj[:, 2 + Q:2 + Q + R].double(), kvw.double(), eps)
    shared = plain.rotate_pairs(proj[:, 2 + Q + R:2 + Q + R + rot].double(), torch.tensor(positions), freq, grow)
    for i, p in enumerate(positions):
        slot = pages[(5 * (p // P) + 1) % npages, p % P].float().cpu()
        close(slot[:R], latent[i], tol, ("latent", p))
        # a 32-bit angle of thousands of radians carries an error of some 1e-4
        close(slot[R:], shared[i], max(tol, 5e-4 if p > 500 else 2e-6), ("rotated key part", p))


@pytest.mark.parametrize("copy_dtype", [None, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,S", [(64, 1), (44, 3), (4096, 2)])
def test_norm_on_a_sublayers_output(W, S, copy_dtype):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(W + S)
    T, eps, mult = 5, 1e-6, 0.35
    x = torch.randn(T, W, generator=g)
    delta = torch.randn(S, T, W, generator=g) * 3.0
    w = (1.0 + 0.3 * torch.randn(W, generator=g)).to(torch.bfloat16)
    want = x.double() + mult * plain.rms_norm(delta.double().sum(0), w.double(), eps)
    for wt in (w.to(DEV), w.float().to(DEV)):
        xd = x.clone().to(DEV)
        copy = torch.empty(T, W, dtype=copy_dtype, device=DEV) if copy_dtype is not None else None
        ops.norm_residual(xd, delta.to(DEV), wt, eps, mult, copy)
        close(xd, want, 2e-6, "stream")
        if copy is not None:
            close(copy.float(), want, 2e-6 if copy_dtype == torch.float32 else 8e-3, "copy")
    # without a sublayer's output only the copy is made
    if copy_dtype is not None:
        xd = x.clone().to(DEV)
        copy = torch.empty(T, W, dtype=copy_dtype, device=DEV)
        ops.norm_residual(xd, None, None, eps, mult, copy)
        assert torch.equal(xd.cpu(), x)
        close(copy.float(), x, 1e-7 if copy_dtype == torch.float32 else 8e-3, "copy alone")


@pytest.mark.parametrize("pairs", [False, True])
def test_feed_forward_gate_of_the_tanh_form(pairs):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, I = 7, 52
    gate, up = 3.0 * torch.randn(T, I, generator=g), torch.randn(T, I, generator=g)
    gu = torch.stack([gate, up], dim=2).reshape(T, 2 * I) if pairs else torch.cat([gate, up], dim=1)
    want = plain.gelu_tanh(gate.double()) * up.double()
    for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
        out = torch.empty(T, I, dtype=dt, device=DEV)
        ops.gated_act(gu.to(DEV), out, "gelu_tanh", pairs=pairs)
        close(out.float(), want, tol, "gate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_query_and_key_norm_with_weights(dtype):
    from allpaca_b200 import ops
    H, G, D, E, P, eps = 3, 1, 24, 40, 8, 1e-5
    g = torch.Generator().manual_seed(2)
    positions = [0, 1, 7, 8, 13, 27]
    T = len(positions)
    qkv = 3.0 * torch.randn(T, (H + G) * D + G * E + H, generator=g)       # the gate's columns behind, not read here
    qw, kw = 1.0 + 0.3 * torch.randn(D, generator=g), 1.0 + 0.3 * torch.randn(D, generator=g)
    pages = torch.zeros(6, G, P, D + E, dtype=dtype, device=DEV)
    bt = i32([[4, 2, 5, 0]])
    q_out = torch.empty(T, H * D, dtype=dtype, device=DEV)
    ops.qk_norm_store(qkv.to(DEV), q_out, pages, i32(positions), i32([0] * T), bt, H, G, D, E, eps, True,
                      q_weight=qw.to(DEV), k_weight=kw.to(DEV))
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    close(q_out.float().view(T, H, D), plain.rms_norm(qkv[:, :H * D].double().view(T, H, D), qw.double(), eps), tol, "queries")
    keys = plain.rms_norm(qkv[:, H * D:(H + G) * D].double().view(T, G, D), kw.double(), eps)
    for i, p in enumerate(positions):
        slot = pages[[4, 2, 5, 0][p // P], :, p % P].float().cpu()
        close(slot[:, :D], keys[i], tol, ("key", p))
        close(slot[:, D:], qkv[i, (H + G) * D:(H + G) * D + G * E].view(G, E), tol, ("value", p))


@pytest.mark.parametrize("H,R,rot,P", [(3, 48, 16, 8), (16, 512, 64, 16), (20, 136, 16, 16), (40, 64, 32, 32), (8, 256, 8, 16)])
@pytest.mark.parametrize("max_context", [1, 4096])
def test_single_rows_in_the_latent_space_on_the_tensor_cores(H, R, rot, P, max_context):
    """Sequences of 1 to 2500 tokens that each bring their last row, beside one that brings two rows (left
    alone): all heads against the shared records, keys cut into one slice or many.  In every sequence
    one head looks hard at one key: the first, the last of a tile of 64, far back."""
    from allpaca_b200 import ops
    from allpaca_b200.parts import Workspace
    g = torch.Generator().manual_seed(H + R)
    D = R + rot
    lens = [1, 64, 65, 2, 700, 2500]
    rows_of = [1, 1, 1, 2, 1, 1]
    scale = 1.0 / math.sqrt(D)
    recs, qs, gates, table, pages_all, want, positions, starts = [], [], [], [], [], [], [], [0]
    base = 0
    for n, rows in zip(lens, rows_of):
        rec = torch.randn(n, D, generator=g).to(torch.bfloat16).double()
        q = torch.randn(rows, H, D, generator=g)
        key = {1: 0, 64: 63, 65: 64, 2: 0, 700: 63, 2500: 1234}[n]
        q[-1, n % H] = 5.0 * math.sqrt(D) * rec[key].float() / rec[key].norm()
        q = q.to(torch.bfloat16).double()
        gate = 2.0 * torch.randn(rows, H, generator=g)
        if rows == 1:
            s = torch.einsum("hd,nd->hn", q[0], rec) * scale
            want.append((torch.softmax(s, dim=-1) @ rec[:, :R]) * torch.sigmoid(gate.double()[0])[:, None])
        else:
            want.append(torch.full((rows, H, R), float("nan"), dtype=torch.float64).view(rows * H, R))
        npg = -(-n // P)
        pg, row = paged(rec[:, None, :], P, shuffled(npg, base))
        pages_all.append(pg[base:, 0])
        table.append(row)
        base += npg
        qs.append(q)
        gates.append(gate)
        positions += list(range(n - rows, n))
        starts.append(starts[-1] + rows)
    pages = torch.cat(pages_all).to(torch.bfloat16).to(DEV)
    width = max(len(r) for r in table)
    bt = i32([r + [-1] * (width - len(r)) for r in table])
    T = starts[-1]
    q = torch.cat(qs).reshape(T, H * D).to(torch.bfloat16).to(DEV).contiguous()
    gate = torch.cat(gates).to(DEV).contiguous()
    out = torch.full((T, H * R), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.latent_decode(q, out, pages, bt, i32(starts), i32(positions), len(lens), H, D, R, scale, gate, max_context,
                      Workspace(torch.device(DEV)))
    got = out.float().cpu().view(T, H, R)
    for s, rows in enumerate(rows_of):
        if rows == 1:
            close(got[starts[s]], want[s], 2e-2, ("sequence of", lens[s]))
        else:
            assert torch.isnan(got[starts[s]:starts[s + 1]]).all(), "rows of a sequence that brings two were written"


@pytest.mark.parametrize("H,DK,DV", [(3, 40, 40), (2, 192, 128), (5, 56, 8), (2, 96, 72), (1, 136, 64)])
def test_prompt_rows_on_per_head_keys_and_values(H, DK, DV):
    """Three sequences in one launch: 70 rows behind 130 earlier tokens, one row (left alone), and 129 rows
    from position 0; per-head keys and values lie token after token.  Chosen rows look hard at one key: the
    first of all, the first and last of a tile of 64, the row itself."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(H + DK)
    lens = [(130, 70), (40, 1), (0, 129)]
    scale = 1.0 / math.sqrt(DK)
    kvs, qs, gates, want, positions, starts, where = [], [], [], [], [], [0], []
    base = 0
    for before, now in lens:
        T = before + now
        q = torch.randn(T, H, DK, generator=g)
        k = torch.randn(T, H, DK, generator=g)
        v = torch.randn(T, H, DV, generator=g)
        gate = 2.0 * torch.randn(T, H, generator=g)
        for row, key in {T - 1: 0, before: min(64, before), T - 2: 63, T - 3: T - 3, before + 1: before}.items():
            if 0 <= key <= row < T and row >= before:
                k[key] = 0.3 * k[key] + 6.0 * q[row] / q[row].norm(dim=-1, keepdim=True) * math.sqrt(DK)
        q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
        s = torch.einsum("ihd,jhd->hij", q, k) * scale
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        full = torch.einsum("hij,jhe->ihe", torch.softmax(s, dim=-1), v) * torch.sigmoid(gate.double())[:, :, None]
        want.append(full[before:])
        qs.append(q[before:])
        gates.append(gate[before:])
        positions += list(range(before, T))
        starts.append(starts[-1] + now)
        if now > 1:
            kvs.append(torch.cat([k, v], dim=-1).reshape(T, H * (DK + DV)))
            where.append(list(range(base, base + T)))
            base += T
        else:
            where.append([])
    width = max(len(w) for w in where)
    wh = i32([w + [-1] * (width - len(w)) for w in where])
    kv = torch.cat(kvs).to(torch.bfloat16).to(DEV).contiguous()
    T = starts[-1]
    q = torch.cat(qs).reshape(T, H * DK).to(torch.bfloat16).to(DEV).contiguous()
    gate = torch.cat(gates).to(DEV).contiguous()
    out = torch.full((T, H * DV), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.latent_prefill_takes(DK, DV)
    ops.latent_prefill(q, out, kv, wh, i32(starts), i32(positions), len(lens), H, DK, DV, scale, gate)
    got = out.float().cpu().view(T, H, DV)
    close(got[:70], want[0], 2e-2, "rows behind earlier tokens")
    close(got[71:], want[2], 2e-2, "rows from position 0")
    assert torch.isnan(got[70]).all(), "the row of a sequence that brings one was written"


@pytest.mark.parametrize("M", [3, 16, 100, 300, 2048])
def test_feed_forward_gate_in_the_products_epilogue(M):
    """The gate-and-up product with the tanh form of GELU applied in its epilogue (few rows, many rows on one SM
    and on a pair of SMs), against the product and the gate computed apart."""
    from allpaca_b200 import ops
    from allpaca_b200.parts import BuildEnv, Workspace
    from allpaca_b200.parts.linear import Linear
    g = torch.Generator().manual_seed(M)
    K, I = 256, 1024
    env = BuildEnv(dtype=torch.bfloat16, device=torch.device(DEV), workspace=Workspace(torch.device(DEV)))
    gate = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16)
    up = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16)
    lin = Linear(env, 2 * I, K)
    lin.load(torch.stack([gate, up], dim=1).reshape(2 * I, K).to(DEV))
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    got = lin.forward_gated(a.to(DEV), "t.act", activation="gelu_tanh")
    assert got is not None
    # the gate and the up value pass through the storage type before the activation
    gt = (a.double() @ gate.double().T).to(torch.bfloat16).double()
    u = (a.double() @ up.double().T).to(torch.bfloat16).double()
    close(got.float(), plain.gelu_tanh(gt) * u, 1e-2, "gated product")
    ops.check_kernel_status()
