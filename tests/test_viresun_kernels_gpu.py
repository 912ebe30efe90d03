"""Each mechanism of the Viresun decoder alone, kernel against the plain implementation, with
inputs made so that a fault shows: one key whose score stands out, far away, just inside and
just outside the window, at page borders, in prompt portions and in single decoded rows;
convolution and recurrence carried over portions shorter than the convolution; state slots that
change hands; routing with distinct logits."""
import math

import pytest
import torch

import plain_viresun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def close(got, want, tol, what):
    got, want = got.double().cpu(), want.double()
    err = float((got - want).abs().max() / want.abs().max().clamp(min=1e-30))
    assert torch.isfinite(got).all() and err <= tol, (what, err)


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_position_vector_and_norm(table_dtype):
    from allpaca_b200 import ops
    V, W, eps = 50, 72, 1e-5
    g = torch.Generator().manual_seed(0)
    table = torch.randn(V, W, generator=g).to(torch.bfloat16).float()
    gain = torch.tensor(1.25)
    tokens = torch.randint(0, V, (9,), generator=g)
    positions = [0, 1, 2, 63, 64, 1000, 4097, 30000, 5]
    want = torch.stack([plain.embed([int(t)] * (p + 1), table.double(), gain.double(), eps)[p]
                        for t, p in zip(tokens, positions)])
    i = torch.arange(W // 2, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * i / W).float().to(DEV)
    x = torch.empty(9, W, device=DEV)
    ops.embed_sinusoid_norm(i32(tokens.tolist()), i32(positions), table.to(table_dtype).to(DEV), inv_freq,
                            gain.expand(W).contiguous().to(DEV), eps, x)
    # a 32-bit angle of 30000 radians carries an error of about 2e-3
    close(x[:7], want[:7], 2e-4, "embedding")
    close(x, want, 3e-3, "embedding at far positions")


def paged(kv, P, order):
    """kv [T, G, D+E] of one sequence -> (pages [n, G, P, D+E], block-table row) with the
    sequence's pages at the places ``order`` names."""
    T, G, F = kv.shape
    n = -(-T // P)
    pages = torch.full((max(order) + 1, G, P, F), float("nan"))
    for b in range(n):
        rows = kv[b * P:(b + 1) * P]
        pages[order[b], :, :rows.shape[0]] = rows.transpose(0, 1)
        pages[order[b], :, rows.shape[0]:] = 0.0
    return pages, order[:n]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,G,D,E,P,window", [(4, 2, 24, 40, 8, 21), (2, 2, 64, 64, 16, 72), (3, 1, 16, 80, 16, None),
                                              (8, 8, 128, 32, 32, 300), (1, 1, 8, 8, 8, 1),
                                              # sizes that are no multiple of 8 (no 16-byte runs), an odd one, more
                                              # than 8 query heads to a key/value head, and heads over 128
                                              (2, 1, 20, 12, 8, 11), (2, 2, 33, 7, 16, 40), (12, 1, 16, 16, 8, 64),
                                              (2, 1, 160, 136, 16, 100)])
def test_attention_with_a_key_that_stands_out(dtype, tol, H, G, D, E, P, window):
    """Two sequences in one launch: a portion of 37 rows behind 300 cached tokens and a single
    decoded row at position 333 of another.  In each, one key is made to dominate for chosen
    rows: far back, at a page's first and last slot, the oldest key the window still shows and the
    one just behind it."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + D)
    lens = [(300, 37), (333, 1)]                       # (cached before, rows now)
    scale = 1.0 / math.sqrt(D)
    r1 = (0.5 + torch.rand(H, generator=g))
    r2 = (0.05 + 0.5 * torch.rand(H, generator=g))
    qs, pages_all, table, want = [], [], [], []
    base = 0
    for s, (before, now) in enumerate(lens):
        T = before + now
        q = torch.randn(T, H, D, generator=g)
        k = torch.randn(T, G, D, generator=g)
        v = torch.randn(T, G, E, generator=g)
        w = window or T
        spikes = {T - 1: T - w, T - 2: T - 2 - w, before: max(0, before - w + 1), before + 1: (before // P) * P,
                  T - 3: ((T - 3 - min(w, T) + 1 + P - 1) // P) * P + P - 1 if w > 2 * P else T - 3}
        for row, key in spikes.items():
            if 0 <= key <= row < T and row >= before:
                # row `row` looks hard at key `key` (if the window shows it)
                k[key] = 0.3 * k[key] + 4.0 * q[row, ::H // G] / q[row, ::H // G].norm(dim=-1, keepdim=True) * math.sqrt(D)
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
        full = plain.biased_window_attention(q.double(), k.double(), v.double(), scale, window, r1.double(), r2.double())
        want.append(full[before:])
        qs.append(q[before:])
        n = -(-T // P)
        order = [base + (7 * b + 3) % n for b in range(n)] if math.gcd(7, n) == 1 else [base + n - 1 - b for b in range(n)]
        pg, row = paged(torch.cat([k, v], dim=-1), P, order)
        pages_all.append(pg[base:])
        table.append(row)
        base += n
    pages = torch.cat(pages_all).to(dtype).to(DEV)
    width = max(len(r) for r in table)
    if window:
        # pages the window has passed were given back: their table entries are void, their contents gone
        for s, (before, now) in enumerate(lens):
            for b in range((before - window + 1) // P if before - window + 1 > 0 else 0):
                pages[table[s][b]] = float("nan")
                table[s][b] = -1
    bt = i32([r + [-1] * (width - len(r)) for r in table])
    q = torch.cat(qs).reshape(-1, H * D).to(dtype).to(DEV).contiguous()
    out = torch.empty(q.shape[0], H * E, dtype=dtype, device=DEV)
    positions = i32([p for before, now in lens for p in range(before, before + now)])
    ops.attention_window_bias(q, out, pages, bt, i32([0, 37, 38]), positions, 2, H, G, D, E, scale, window or 0,
                              r1.to(DEV), r2.to(DEV))
    close(out.float().reshape(-1, H, E), torch.cat(want), tol, "attention")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_query_and_key_norm_temperature_and_store(dtype):
    from allpaca_b200 import ops
    H, G, D, E, P, eps = 3, 1, 24, 40, 8, 1e-5
    g = torch.Generator().manual_seed(2)
    positions = [0, 1, 6, 7, 8, 13, 14, 27, 28]          # temperature steps at 6, 13, 27 (every 7)
    T = len(positions)
    qkv = 3.0 * torch.randn(T, (H + G) * D + G * E, generator=g)
    pages = torch.zeros(6, G, P, D + E, dtype=dtype, device=DEV)
    bt = i32([[4, 2, 5, 0]])
    q_out = torch.empty(T, H * D, dtype=dtype, device=DEV)
    ops.qk_norm_store(qkv.to(DEV), q_out, pages, i32(positions), i32([0] * T), bt, H, G, D, E, eps, True, 0.4, 7)
    qw = plain.unit_rms(qkv[:, :H * D].double().view(T, H, D), eps)
    temp = torch.tensor([1 + 0.4 * math.log((p + 1) // 7 + 1) for p in positions], dtype=torch.float64)
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    close(q_out.float().view(T, H, D), qw * temp[:, None, None], tol, "queries")
    kw = plain.unit_rms(qkv[:, H * D:(H + G) * D].double().view(T, G, D), eps)
    for i, p in enumerate(positions):
        slot = pages[[4, 2, 5, 0][p // P], :, p % P].float().cpu()
        close(slot[:, :D], kw[i], tol, ("key", p))
        close(slot[:, D:], qkv[i, (H + G) * D:].view(G, E), tol, ("value", p))


@pytest.mark.parametrize("taps,C", [(4, 37), (2, 64), (3, 300), (1, 5)])
def test_convolution_carried_over_portions(taps, C):
    """Two sequences in alternating slots, cut into portions of 1, 2, 1, 5, 3 ... rows (shorter than
    the convolution), each step one launch over both."""
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(taps)
    L = [23, 17]
    u = [torch.randn(n, C + 6, generator=g) for n in L]
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    want = [plain.silu(plain.causal_conv(x[:, 4:4 + C].double(), w.double(), b.double())) for x in u]
    state = torch.full((3, max(taps - 1, 1), C), float("nan"), device=DEV)      # slots 2 and 0 are used
    got = [[], []]
    at = [0, 0]
    cuts = [1, 2, 1, 5, 3, 1, 1, 7, 2, 30]
    k = 0
    while at[0] < L[0] or at[1] < L[1]:
        rows, seqs = [], []
        for s in (0, 1):
            n = min(cuts[(k + s) % len(cuts)], L[s] - at[s])
            if n > 0:
                seqs.append((s, at[s], n))
                rows.append(u[s][at[s]:at[s] + n])
        k += 1
        x = torch.cat(rows).to(DEV).contiguous()
        T = x.shape[0]
        starts = [0]
        for _, _, n in seqs:
            starts.append(starts[-1] + n)
        out = torch.empty(T, C, device=DEV)
        ops.causal_conv_silu(x, 4, w.to(DEV), b.to(DEV), state if taps > 1 else None,
                             i32([j for j, (_, _, n) in enumerate(seqs) for _ in range(n)]), i32(starts),
                             i32([a + i for _, a, n in seqs for i in range(n)]), i32([2 if s == 0 else 0 for s, _, _ in seqs]),
                             out, len(seqs))
        for j, (s, a, n) in enumerate(seqs):
            got[s].append(out[starts[j]:starts[j + 1]].cpu())
            at[s] += n
    for s in (0, 1):
        close(torch.cat(got[s]), want[s], 2e-6, ("convolution", s))


@pytest.mark.parametrize("Hh,E,N,G", [(6, 12, 20, 3), (4, 32, 70, 1), (2, 64, 128, 2), (3, 5, 3, 3), (1, 100, 16, 1)])
def test_recurrence_carried_over_portions_and_slots(Hh, E, N, G):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(Hh * 10 + N)
    inner = Hh * E

    def sequence(n):
        return torch.randn(n, inner + 2 * G * N, generator=g), torch.randn(n, Hh + 3, generator=g)
    a_log = torch.log(0.02 + 0.3 * torch.rand(Hh, generator=g))
    dt_bias, d_skip = torch.randn(Hh, generator=g) - 0.5, torch.randn(Hh, generator=g)

    def want(xbc, dt):
        return plain.ssm_recurrence(xbc[:, :inner].double().view(-1, Hh, E), xbc[:, inner:inner + G * N].double().view(-1, G, N),
                                    xbc[:, inner + G * N:].double().view(-1, G, N),
                                    torch.log1p(torch.exp(dt[:, 3:].double() + dt_bias.double())), a_log.double(),
                                    d_skip.double()).reshape(-1, inner)
    state = torch.full((2, Hh, N, E), float("nan"), device=DEV)
    args = (dt_bias.to(DEV), a_log.to(DEV), d_skip.to(DEV), state)

    def run(parts):
        """parts: (xbc rows, dt rows, first position, slot) per sequence of the step."""
        xbc = torch.cat([p[0] for p in parts]).to(DEV).contiguous()
        dt = torch.cat([p[1] for p in parts]).to(DEV).contiguous()
        starts = [0]
        for p in parts:
            starts.append(starts[-1] + p[0].shape[0])
        y = torch.empty(xbc.shape[0], inner, device=DEV)
        ops.ssm_scan(xbc, dt[:, 3:], *args, i32(starts), i32([p[2] + i for p in parts for i in range(p[0].shape[0])]),
                     i32([p[3] for p in parts]), y, len(parts), Hh, G, N, E)
        return [y[starts[j]:starts[j + 1]].cpu() for j in range(len(parts))]
    xa, da = sequence(41)
    xb, db = sequence(9)
    ya, yb = [], []
    r = run([(xa[:17], da[:17], 0, 1), (xb[:1], db[:1], 0, 0)]); ya.append(r[0]); yb.append(r[1])
    r = run([(xb[1:3], db[1:3], 1, 0), (xa[17:18], da[17:18], 17, 1)]); yb.append(r[0]); ya.append(r[1])
    r = run([(xa[18:], da[18:], 18, 1), (xb[3:], db[3:], 3, 0)]); ya.append(r[0]); yb.append(r[1])
    close(torch.cat(ya), want(xa, da), 2e-5, "recurrence, long sequence")
    close(torch.cat(yb), want(xb, db), 2e-5, "recurrence, short sequence")
    # slot 1 changes hands: a new sequence starts at position 0 there, nothing of the old one is left
    xc, dc = sequence(5)
    close(run([(xc, dc, 0, 1)])[0], want(xc, dc), 2e-5, "recurrence in a slot used before")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_then_norm_in_parts(dtype):
    from allpaca_b200 import ops
    g = torch.Generator().manual_seed(5)
    T, inner, parts, eps = 7, 72, 3, 1e-5
    y, z = torch.randn(T, inner, generator=g), torch.randn(T, inner + 9, generator=g)
    w = (1 + 0.2 * torch.randn(inner, generator=g)).to(dtype)
    gated = y.double() * plain.silu(z[:, 2:2 + inner].double())
    want = plain.unit_rms(gated.view(T, parts, inner // parts), eps).reshape(T, inner) * w.double()
    out = torch.empty(T, inner, dtype=dtype, device=DEV)
    ops.gated_group_rmsnorm(y.to(DEV), z.to(DEV)[:, 2:2 + inner], w.to(DEV), eps, out, parts)
    close(out.float(), want, 2e-6 if dtype == torch.float32 else 8e-3, "gated norm")


def test_routing_and_grouping():
    from allpaca_b200 import ops
    T, E, top = 77, 11, 3
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(T, E, generator=g)
    logits[5] = 0.0                                       # all equal: the lowest indices win
    bias = torch.randn(E, generator=g)
    chosen = torch.empty(T, top, dtype=torch.int32, device=DEV)
    weight = torch.empty(T, top, device=DEV)
    ops.moe_route(logits.to(DEV), bias.to(DEV), chosen, weight)
    best, idx = torch.topk((logits + bias).double(), top, dim=1)
    assert torch.equal(chosen.cpu().long(), idx)
    close(weight, torch.softmax(best, dim=1), 1e-6, "routing weights")
    pairs = T * top
    perm = torch.empty(pairs, dtype=torch.int32, device=DEV)
    place = torch.empty(pairs, dtype=torch.int32, device=DEV)
    tiles = torch.zeros(ops.moe_max_tiles(pairs, E) + 1, 3, dtype=torch.int32, device=DEV)
    ops.moe_sort(chosen, perm, place, tiles, E)
    perm, place, tiles = perm.cpu().long(), place.cpu().long(), tiles.cpu().long()
    assert sorted(perm.tolist()) == list(range(pairs)) and torch.equal(perm[place], torch.arange(pairs))
    experts = chosen.cpu().long().reshape(-1)[perm]
    assert torch.equal(experts, experts.sort().values)    # grouped by expert
    covered = []
    for e, first, rows in tiles[:int(tiles[-1, 0])].tolist():
        assert 0 < rows <= 64 and (experts[first:first + rows] == e).all()
        covered += list(range(first, first + rows))
    assert covered == list(range(pairs))


def build_part(kind, name, params, tensors, dtype):
    from allpaca_b200.parts import BuildEnv, PartSpec, Workspace, build
    dev = torch.device(DEV)
    part = build(kind, PartSpec(name, params), BuildEnv(dtype, dev, Workspace(dev)))
    part.load({k: v.to(dtype).to(dev) for k, v in tensors.items()})
    return part


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("W,F,E,top,T", [(72, 40, 6, 2, 150), (128, 64, 9, 3, 5), (40, 24, 5, 1, 70), (64, 96, 4, 4, 1)])
def test_routed_feed_forward(dtype, tol, W, F, E, top, T):
    g = torch.Generator().manual_seed(W + E)
    w = {"router": torch.randn(E, W, generator=g), "router.b": torch.randn(E, generator=g)}
    for e in range(E):
        w.update({f"e{e}.gate": torch.randn(F, W, generator=g) * 0.25, f"e{e}.up": torch.randn(F, W, generator=g) * 0.25,
                  f"e{e}.down": torch.randn(W, F, generator=g) * 0.2})
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    h = torch.randn(T, W, generator=g).to(dtype)
    part = build_part("feed_forward", "routed_experts", {"hidden_size": W, "expert_size": F, "experts": E, "top": top,
                                                         "limit": 1.25}, w, dtype)
    got = part.forward(h.to(DEV), None).sum(0)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": F, "limit": 1.25}}
    want = plain.routed_feed_forward(h.double(), {"x." + k: v.double() for k, v in w.items()}, "x.", mlp)
    close(got, want, tol, "routed feed-forward")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_dense_feed_forward_with_relu_gate(dtype, tol):
    g = torch.Generator().manual_seed(3)
    W, F, T = 72, 88, 19
    w = {"gate": torch.randn(F, W, generator=g) * 0.2, "up": torch.randn(F, W, generator=g) * 0.2,
         "down": torch.randn(W, F, generator=g) * 0.2}
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    h = torch.randn(T, W, generator=g).to(dtype)
    part = build_part("feed_forward", "swiglu", {"hidden_size": W, "intermediate_size": F, "activation": "relu",
                                                 "names": ("gate", "up", "down")}, w, dtype)
    got = part.forward(h.to(DEV), None).sum(0)
    want = plain.dense_feed_forward(h.double(), {"x." + k: v.double() for k, v in w.items()}, "x.")
    close(got, want, tol, "dense feed-forward")
