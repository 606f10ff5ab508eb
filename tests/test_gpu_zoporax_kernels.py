"""The kernels that the Zoporax design added, each alone against a float64 restatement of its own operation
written here: the latent cache write, the rotation of a head's tail, per-head matrices, attention over latent
rows (window edges, page borders, a far key, the first tokens, shuffled pages with NaN elsewhere, sliced keys),
the router, the experts' products, the gated activation, and the scan with silu on its inputs."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from longbow_quarrel_b200.kernels import ops
    return ops


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _tables(dims, n_pos, base=100.0, mult=1.0):
    f = torch.tensor(base, dtype=torch.float64) ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    a = torch.arange(n_pos, dtype=torch.float64)[:, None] * f
    return (torch.cos(a) * mult).float().to(DEV).contiguous(), (torch.sin(a) * mult).float().to(DEV).contiguous()


def _rotate(x, pos, cos, sin, rot):
    """float64 reference: x [..., n], first `rot` dimensions rotated by the tables' row `pos`."""
    half = rot // 2
    c, s = cos[pos].double().cpu(), sin[pos].double().cpu()
    u, v = x[..., :half], x[..., half:rot]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., rot:]], dim=-1)


def _rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).norm() / ref.norm().clamp_min(1e-30))


# ------------------------------------------------------------------ cache write, rotation, per-head matrices

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,dr,rot", [(24, 8, 8), (20, 12, 8), (96, 24, 24), (36, 4, 0)])
def test_latent_rows_are_normed_rotated_and_stored_in_their_pages(dtype, R, dr, rot):
    ops = _ops()
    g = torch.Generator().manual_seed(R)
    page_size, T = 8, 13
    rows = torch.randn(T, 5 + R + dr + 3, generator=g)
    gain = (1 + 0.3 * torch.randn(R, generator=g)).float()
    cos, sin = _tables(rot, 64) if rot else (None, None)
    # Two sequences in slots 2 and 0: positions 5..11 of one, 0..5 of the other, pages handed out in a shuffled order.
    pos = list(range(5, 12)) + list(range(0, 6))
    seq = [0] * 7 + [1] * 6
    table = torch.full((3, 4), -1, dtype=torch.int32)
    table[2, :2] = torch.tensor([3, 1])
    table[0, :1] = torch.tensor([4])
    pages = torch.full((6, page_size, R + dr), float("nan"), dtype=dtype, device=DEV)
    ops.latent_kv_store(rows.to(DEV), 5, 5 + R, gain.to(DEV), 1e-5, cos, sin, rot, _i32(pos), _i32(seq), _i32([2, 0]),
                        table.to(DEV), pages, R, dr, page_size)
    got = pages.float().cpu()
    x = rows.double()
    written = set()
    for t in range(T):
        c = x[t, 5:5 + R]
        ref = torch.cat([c / torch.sqrt((c * c).mean() + 1e-5) * gain.double(),
                         _rotate(x[t, 5 + R:5 + R + dr], pos[t], cos, sin, rot) if rot else x[t, 5 + R:5 + R + dr]])
        page = int(table[[2, 0][seq[t]], pos[t] // page_size])
        written.add((page, pos[t] % page_size))
        assert _rel(got[page, pos[t] % page_size], ref) < (1e-6 if dtype == torch.float32 else 4e-3), t
    untouched = [(p, r) for p in range(6) for r in range(page_size) if (p, r) not in written]
    assert all(torch.isnan(got[p, r]).all() for p, r in untouched)


@pytest.mark.parametrize("src_dtype", [torch.float32, torch.bfloat16])
def test_the_tail_of_every_head_is_rotated_into_the_wide_query(src_dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    T, H, dn, dr, R, rot = 9, 3, 10, 12, 7, 8
    q = torch.randn(T, H * (dn + dr), generator=g).to(src_dtype)
    cos, sin = _tables(rot, 300, mult=1.07)
    pos = [0, 1, 2, 100, 101, 299, 7, 8, 9]
    wide = torch.zeros(T, H * (R + dr), device=DEV)
    ops.rope_tail(q.to(DEV), dn + dr, dn, wide, R + dr, R, cos, sin, rot, _i32(pos), H, dr)
    qd = q.double().reshape(T, H, dn + dr)
    for t in range(T):
        ref = _rotate(qd[t, :, dn:], pos[t], cos, sin, rot)
        assert _rel(wide[t].reshape(H, R + dr)[:, R:], ref) < 1e-6
    assert float(wide.reshape(T, H, R + dr)[:, :, :R].abs().max()) == 0.0


@pytest.mark.parametrize("in_dtype,w_dtype,out_dtype", [(torch.float32, torch.float32, torch.float32),
                                                        (torch.float32, torch.bfloat16, torch.float32),
                                                        (torch.float32, torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("T,H,K,N", [(1, 1, 8, 5), (13, 3, 24, 40), (70, 8, 32, 96), (9, 2, 300, 17)])
def test_one_matrix_per_head(in_dtype, w_dtype, out_dtype, T, H, K, N):
    ops = _ops()
    g = torch.Generator().manual_seed(T + K)
    src = torch.randn(T, H * (K + 3) + 2, generator=g).to(in_dtype)
    w = (torch.randn(H, K, N, generator=g) / math.sqrt(K)).to(w_dtype)
    out = torch.full((T, H * (N + 4)), 7.0, dtype=out_dtype, device=DEV)
    ops.head_matmul(src.to(DEV), K + 3, 2, w.to(DEV), out, N + 4, 1)
    ref = torch.einsum("thk,hkn->thn", src.double()[:, :H * (K + 3)].reshape(T, H, K + 3)[:, :, 2:2 + K], w.double())
    got = out.reshape(T, H, N + 4)
    assert _rel(got[:, :, 1:1 + N], ref) < (2e-6 if out_dtype == torch.float32 else 4e-3)
    assert (got[:, :, 0] == 7.0).all() and (got[:, :, 1 + N:] == 7.0).all()          # nothing beside its columns


# ------------------------------------------------------------------ the attention

def _latent_reference(q, rows, pos, window, R, scale):
    """q [H, Dk] float64, rows [n, Dk] the sequence's latent rows: softmax over the window, mean of the rows' first R."""
    first = 0 if not window else max(0, pos - window + 1)
    keys = rows[first:pos + 1]
    p = torch.softmax(keys @ q.T * scale, dim=0)            # [keys, H]
    return p.T @ keys[:, :R]


def _paged(rows_by_seq, Dk, page_size, dtype, n_pages, seed):
    """The sequences' rows laid into pages in a shuffled order, NaN everywhere else; returns (pages, table)."""
    order = np.random.default_rng(seed).permutation(n_pages).tolist()
    pages = torch.full((n_pages, page_size, Dk), float("nan"), dtype=dtype)
    most = max(-(-len(r) // page_size) for r in rows_by_seq.values())
    table = torch.full((max(rows_by_seq) + 1, most), -1, dtype=torch.int32)
    for slot, rows in rows_by_seq.items():
        for p in range(-(-len(rows) // page_size)):
            page = order.pop()
            table[slot, p] = page
            chunk = rows[p * page_size:(p + 1) * page_size]
            pages[page, :len(chunk)] = chunk.to(dtype)
    return pages.to(DEV), table.to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,dr,window,splits", [(3, 24, 8, 33, 1), (1, 20, 12, None, 1), (8, 96, 24, 64, 1), (9, 40, 16, 100, 3),
                                                  (2, 300, 20, 5, 1), (4, 16, 8, 64, 4)])
def test_attention_over_latent_rows(dtype, H, R, dr, window, splits):
    """Rows of three sequences in one launch: whole prompts from the first token, positions on both sides of page
    borders and of the window's edge, and single late rows."""
    ops = _ops()
    g = torch.Generator().manual_seed(H * 100 + R)
    Dk, page_size = R + dr, 16
    lens = {0: 150, 2: 70, 3: 17}
    rows = {s: torch.randn(n, Dk, generator=g) for s, n in lens.items()}
    pages, table = _paged(rows, Dk, page_size, dtype, 20, seed=H)
    stored = {s: r.to(dtype).double() for s, r in rows.items()}
    slots = [2, 0, 3]
    w = window or 0
    # sequence 0 of the step (slot 2): its whole prompt; sequence 1 (slot 0): late rows around borders and the window; sequence 2: its last
    pos = list(range(70)) + [15, 16, 17, 31, 32, 47, 48, 63, 64, 65, 99, 100, 101, 127, 128, 149] + [16]
    seq = [0] * 70 + [1] * 16 + [2]
    if w:
        pos += [w - 2, w - 1, w, w + 1]
        seq += [1] * 4
    T = len(pos)
    q = torch.randn(T, H, Dk, generator=g)
    out = ops.latent_attention(q.to(DEV), pages, table, _i32(pos), _i32(seq), _i32(slots), H, R, page_size, 0.2, window, splits)
    tol = 3e-6 if dtype == torch.float32 else 3e-6          # the reference reads the rounded cache rows: only sums differ
    for t in range(T):
        ref = _latent_reference(q[t].double(), stored[slots[seq[t]]], pos[t], w, R, 0.2)
        assert _rel(out[t], ref) < tol, (t, pos[t], seq[t])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [40, 64, 257])
@pytest.mark.parametrize("splits", [1, 5])
def test_a_key_that_outweighs_all_others_just_inside_and_just_outside_the_window(dtype, window, splits):
    """One cached row is made to match the query a hundred times better than the rest.  At the last position that
    still sees it the output must be that row; one position later nothing of it may be left; and a row far back
    (hundreds of keys away, across many pages) is found whole when there is no window."""
    ops = _ops()
    g = torch.Generator().manual_seed(window)
    H, R, dr, page_size = 2, 32, 8, 64
    Dk = R + dr
    n = 700
    rows = 0.1 * torch.randn(n, Dk, generator=g)
    planted = 300
    direction = torch.randn(Dk, generator=g)
    direction /= direction.norm()
    rows[planted] = 8.0 * direction
    pages, table = _paged({1: rows}, Dk, page_size, dtype, 12, seed=window)
    stored = rows.to(dtype).double()
    pos = [planted, planted + 1, planted + window - 2, planted + window - 1, planted + window, planted + window + 1, n - 1]
    q = (8.0 * direction).repeat(len(pos), H, 1)
    for win in (window, None):
        out = ops.latent_attention(q.to(DEV), pages, table, _i32(pos), _i32([0] * len(pos)), _i32([1]), H, R, page_size, 1.0,
                                   win, splits)
        for t, p in enumerate(pos):
            ref = _latent_reference(q[t].double(), stored, p, win or 0, R, 1.0)
            assert _rel(out[t], ref) < 1e-5, (win, p)
            sees = win is None or p - planted < win
            closeness = _rel(out[t, 0], stored[planted, :R])
            assert (closeness < 1e-3) == sees, (win, p, closeness)


# ------------------------------------------------------------------ routed experts

def _route_reference(z, E, groups, keep, top, scale):
    s = torch.sigmoid(z.double())
    per = E // groups
    gs = s.reshape(groups, per).topk(min(2, per), dim=1).values.sum(dim=1)
    allowed = torch.zeros(E, dtype=torch.bool)
    for gidx in gs.topk(keep).indices.tolist():
        allowed[gidx * per:(gidx + 1) * per] = True
    chosen = torch.where(allowed, s, torch.full_like(s, -1.0)).topk(top).indices
    return chosen.tolist(), (s[chosen] / (s[chosen].sum() + 1e-20) * scale)


@pytest.mark.parametrize("E,groups,keep,top", [(8, 4, 1, 2), (6, 3, 2, 2), (16, 4, 2, 3), (5, 1, 1, 2), (3, 1, 1, 3), (64, 8, 3, 6),
                                               (4, 4, 2, 1), (160, 8, 3, 6)])
def test_the_router_chooses_by_groups(E, groups, keep, top):
    ops = _ops()
    g = torch.Generator().manual_seed(E * 10 + top)
    T = 50
    z = 2.0 * torch.randn(T, E + 1, generator=g)          # one more column rides along (another gate's logit)
    ids, weights = ops.moe_route(z.to(DEV), E, groups, keep, top, 1.7)
    ids, weights = ids.cpu(), weights.double().cpu()
    for t in range(T):
        chosen, ref = _route_reference(z[t, :E], E, groups, keep, top, 1.7)
        assert ids[t].tolist() == chosen, t                  # in the order of their scores
        assert (weights[t] - ref).abs().max() < 1e-6


def test_the_router_leaves_the_best_expert_when_its_group_loses():
    ops = _ops()
    s = torch.tensor([[0.95, 0.05, 0.6, 0.55, 0.1, 0.2]])
    z = torch.log(s / (1 - s))
    ids, weights = ops.moe_route(z.to(DEV), 6, 3, 1, 2, 2.0)
    assert sorted(ids[0].tolist()) == [2, 3] and float(weights.sum()) == pytest.approx(2.0, rel=1e-6)
    ids, _ = ops.moe_route(z.to(DEV), 6, 3, 2, 2, 2.0)
    assert sorted(ids[0].tolist()) == [0, 2]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,D,F", [(1, 3, 3, 40, 16), (37, 8, 2, 64, 24), (5, 16, 3, 100, 50), (300, 6, 1, 128, 48)])
def test_the_experts_products_and_the_shared_rows_join_the_stream(dtype, T, E, top, D, F):
    ops = _ops()
    g = torch.Generator().manual_seed(T + E)
    h = torch.randn(T, D, generator=g).to(dtype)
    w_up = (torch.randn(E, F, D, generator=g) / math.sqrt(D)).to(dtype)
    w_down = (torch.randn(E, D, F, generator=g) / math.sqrt(F)).to(dtype)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    weights = torch.rand(T, top, generator=g)
    shared = torch.randn(T, D, generator=g)
    zs = torch.randn(T, 3, generator=g)
    x0 = torch.randn(T, D, generator=g)
    u = ops.moe_up(h.to(DEV), w_up.to(DEV), ids.to(DEV), "gelu")
    pre = torch.einsum("tjfd,td->tjf", w_up.double()[ids.long()], h.double())
    u_ref = 0.5 * pre * (1 + torch.erf(pre / math.sqrt(2.0)))
    assert _rel(u, u_ref) < (2e-6 if dtype == torch.float32 else 4e-3)
    x = x0.clone().to(DEV)
    ops.moe_down(u, w_down.to(DEV), ids.to(DEV), weights.to(DEV), x, True, shared.to(DEV), zs.to(DEV)[:, 1])
    y = torch.einsum("tjdf,tjf->tjd", w_down.double()[ids.long()], u.double().cpu())
    ref = x0.double() + (weights.double()[:, :, None] * y).sum(1) + torch.sigmoid(zs[:, 1].double())[:, None] * shared.double()
    assert _rel(x, ref) < 2e-6
    out = torch.empty(T, D, device=DEV)
    ops.moe_down(u, w_down.to(DEV), ids.to(DEV), weights.to(DEV), out, False)
    assert _rel(out, (weights.double()[:, :, None] * y).sum(1)) < 2e-6


# ------------------------------------------------------------------ element by element

@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                                (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("kind", ["gelu_tanh", "gelu", "silu"])
def test_gated_activation_with_biases(in_dtype, out_dtype, kind):
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    T, F = 11, 50
    gu = (2 * torch.randn(T, 2 * F, generator=g)).to(in_dtype)
    bias = torch.randn(2 * F, generator=g)
    acts = {"gelu_tanh": lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))),
            "gelu": lambda z: 0.5 * z * (1 + torch.erf(z / math.sqrt(2.0))), "silu": lambda z: z * torch.sigmoid(z)}
    for b in (bias, None):
        out = ops.gated_act(gu.to(DEV), b.to(DEV) if b is not None else None, kind, out_dtype)
        x = gu.double() + (b.double() if b is not None else 0.0)
        ref = acts[kind](x[:, :F]) * x[:, F:]
        assert _rel(out, ref) < (2e-6 if out_dtype == torch.float32 else 4e-3)
    x = torch.randn(T, F, generator=g)
    got = ops.add_bias(x.clone().to(DEV), bias[:F].to(DEV))
    assert _rel(got, x.double() + bias[:F].double()) < 1e-7
    y = torch.randn(T, F, generator=g).to(in_dtype)
    assert _rel(ops.activation(y.to(DEV), "gelu"), acts["gelu"](y.double())) < (2e-6 if in_dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv", [(2, 16, 24), (1, 40, 12), (4, 64, 64)])
def test_the_scan_with_silu_on_its_inputs_in_pieces_and_single_tokens(dtype, H, dk, dv):
    """S_t = g S_(t-1) + silu(k_t) silu(v_t)^T, o_t = S_t^T silu(q_t): a prompt in one piece, in pieces of 2, 1, 30 and
    the rest, and token by token, from a first token that must last (decay one on the last head)."""
    ops = _ops()
    g = torch.Generator().manual_seed(dk)
    n = 90
    rows = torch.randn(n, 2 * H * dk + H * dv + 5, generator=g).to(dtype)
    rows[0] *= 4.0
    decay = torch.tensor([0.9, 0.97, 0.5, 1.0][-H:], dtype=torch.float32)
    x = rows.double()
    act = lambda z: z * torch.sigmoid(z)
    q = act(x[:, :H * dk]).reshape(n, H, dk)
    k = act(x[:, H * dk:2 * H * dk]).reshape(n, H, dk)
    v = act(x[:, 2 * H * dk:2 * H * dk + H * dv]).reshape(n, H, dv)
    S = torch.zeros(H, dk, dv, dtype=torch.float64)
    ref = torch.zeros(n, H, dv, dtype=torch.float64)
    for t in range(n):
        S = decay.double()[:, None, None] * S + k[t, :, :, None] * v[t, :, None, :]
        ref[t] = torch.einsum("hkv,hk->hv", S, q[t])
    dev_rows = rows.to(DEV)
    for pieces in ([n], [2, 1, 30, n - 33], [1] * n):
        state = torch.zeros(3, H, dk, dv, device=DEV)
        got, at = [], 0
        for m in pieces:
            out, _ = ops.linear_scan(dev_rows[at:at + m], 0, H * dk, 2 * H * dk, state, _i32([0, m]), _i32([1]),
                                     _i32(list(range(at, at + m))), 1, H, dk, dv, decay=decay.to(DEV), single=(m == 1), in_act="silu")
            got.append(out)
            at += m
        assert _rel(torch.cat(got), ref) < 1e-5, pieces[:3]
        assert _rel(state[1], S) < 1e-5 and float(state[0].abs().max()) == 0.0


# ------------------------------------------------------------------ the attention on the tensor cores

def _blocks_for(new, past, size):
    """The work list of a step whose sequences bring `new` tokens after `past`: the framework's own builder."""
    from longbow_quarrel_b200.kernels.attention import query_blocks
    from longbow_quarrel_b200.parts.base import StepShape
    cu = np.concatenate([[0], np.cumsum(new)])
    flat = query_blocks(size)(StepShape(B=len(new), T=int(sum(new)), past=tuple(past), new=tuple(new), cu=tuple(int(c) for c in cu)))
    return tuple(_i32(row.tolist()) for row in flat)


@pytest.mark.parametrize("H,R,dr,window", [(3, 24, 8, 33), (1, 20, 12, None), (8, 96, 24, 64), (9, 40, 16, 100), (16, 300, 20, 70),
                                           (70, 16, 8, 64), (4, 512, 64, 150)])
def test_tensor_core_attention_over_latent_rows_prompts_portions_and_single_tokens(H, R, dr, window):
    """Three sequences in one launch: a whole prompt from its first token, a portion that goes on after 83 cached tokens
    (across page borders and the window's edge), a short prompt; then single tokens with their keys cut into slices.
    Against a float64 restatement that reads the same rounded queries and cache rows."""
    ops = _ops()
    g = torch.Generator().manual_seed(H * 100 + R)
    Dk, page_size = R + dr, 64
    lens = {0: 200, 2: 70, 3: 17}
    rows = {s: torch.randn(n, Dk, generator=g) for s, n in lens.items()}
    pages, table = _paged(rows, Dk, page_size, torch.bfloat16, 9, seed=H)
    stored = {s: r.to(torch.bfloat16).double() for s, r in rows.items()}
    slots = [2, 0, 3]
    w = window or 0
    new, past = [70, 117, 17], [0, 83, 0]
    pos = [p for n, b in zip(new, past) for p in range(b, b + n)]
    seq = [i for i, n in enumerate(new) for _ in range(n)]
    T = len(pos)
    q = torch.randn(T, H, Dk, generator=g)
    qr = q.to(torch.bfloat16).double()
    out = ops.latent_attention_tc(q.to(DEV), pages, table, _i32(slots), H, R, page_size, 0.2, window,
                                  blocks=_blocks_for(new, past, ops.latent_tc_tokens(H)))
    for t in range(T):
        ref = _latent_reference(qr[t], stored[slots[seq[t]]], pos[t], w, R, 0.2)
        assert _rel(out[t], ref) < 6e-3, (t, pos[t], seq[t])
    # single tokens: the last row of each sequence, and one in the middle of the long one
    for splits in (1, 3):
        pos1, seq1 = [199, 69, 16], [1, 0, 2]
        q1 = torch.randn(3, H, Dk, generator=g)
        out = ops.latent_attention_tc(q1.to(DEV), pages, table, _i32(slots), H, R, page_size, 0.2, window, tok_pos=_i32(pos1),
                                      tok_seq=_i32(seq1), splits=splits)
        for t in range(3):
            ref = _latent_reference(q1[t].to(torch.bfloat16).double(), stored[slots[seq1[t]]], pos1[t], w, R, 0.2)
            assert _rel(out[t], ref) < 6e-3, (splits, t)


@pytest.mark.parametrize("window", [40, 64, 257])
@pytest.mark.parametrize("splits", [1, 5])
def test_tensor_core_attention_finds_the_key_that_outweighs_all_others_up_to_the_window_edge(window, splits):
    ops = _ops()
    g = torch.Generator().manual_seed(window)
    H, R, dr, page_size = 2, 32, 8, 64
    Dk, n, planted = R + dr, 700, 300
    rows = 0.1 * torch.randn(n, Dk, generator=g)
    direction = torch.randn(Dk, generator=g)
    direction /= direction.norm()
    rows[planted] = 8.0 * direction
    pages, table = _paged({1: rows}, Dk, page_size, torch.bfloat16, 12, seed=window)
    stored = rows.to(torch.bfloat16).double()
    # as a portion of a prompt: positions planted .. planted + window + 1 in one step; as single tokens: the edge itself
    first, count = planted, window + 2
    q = (8.0 * direction).repeat(count, H, 1)
    for win in (window, None):
        out = ops.latent_attention_tc(q.to(DEV), pages, table, _i32([1]), H, R, page_size, 1.0, win,
                                      blocks=_blocks_for([count], [first], ops.latent_tc_tokens(H)))
        edge = [(window - 1, True), (window, win is None), (window + 1, win is None), (0, True), (1, True)]
        for off, sees in edge:
            closeness = _rel(out[off, 0], stored[planted, :R])
            assert (closeness < 1e-2) == sees, (win, off, closeness)
        pos1 = [planted + window - 1, planted + window, n - 1]
        out = ops.latent_attention_tc(q[:3].to(DEV), pages, table, _i32([1]), H, R, page_size, 1.0, win, tok_pos=_i32(pos1),
                                      tok_seq=_i32([0, 0, 0]), splits=splits)
        for t, sees in enumerate([True, win is None, win is None]):
            closeness = _rel(out[t, 0], stored[planted, :R])
            assert (closeness < 1e-2) == sees, (win, pos1[t], closeness)


# ------------------------------------------------------------------ many small products in one launch

@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,K,N", [(1, 1, 8, 5), (13, 3, 24, 40), (70, 8, 32, 96), (200, 2, 304, 130), (8, 16, 128, 512)])
def test_one_matrix_per_head_on_the_tensor_cores(out_dtype, T, H, K, N):
    ops = _ops()
    g = torch.Generator().manual_seed(T + K)
    src = torch.randn(T, H * (K + 8), generator=g).to(torch.bfloat16)
    w = (torch.randn(H, N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    out = torch.full((T, H * (N + 3) + 2), 7.0, dtype=out_dtype, device=DEV)
    ops.grouped_gemm(src.to(DEV), w.to(DEV), out, a_group_stride=K + 8, o_group_stride=N + 3)
    ref = torch.einsum("thk,hnk->thn", src.double().reshape(T, H, K + 8)[:, :, :K], w.double())
    got = out[:, :H * (N + 3)].reshape(T, H, N + 3)
    assert _rel(got[:, :, :N], ref) < (2e-6 if out_dtype == torch.float32 else 4e-3)
    assert (got[:, :, N:] == 7.0).all() and (out[:, H * (N + 3):] == 7.0).all()


@pytest.mark.parametrize("T,E,top,D,F", [(40, 3, 3, 40, 16), (137, 8, 2, 64, 24), (300, 16, 3, 104, 56), (300, 6, 1, 128, 48), (64, 160, 6, 64, 32)])
def test_the_experts_products_as_grouped_products(T, E, top, D, F):
    """The (token, choice) pairs sorted by expert on the device, both products as grouped launches, the combination: against
    the same sums in float64 (and so against the kernels that stream every token's own experts)."""
    ops = _ops()
    g = torch.Generator().manual_seed(T + E)
    h = torch.randn(T, D, generator=g).to(torch.bfloat16)
    w_up = (torch.randn(E, F, D, generator=g) / math.sqrt(D)).to(torch.bfloat16)
    w_down = (torch.randn(E, D, F, generator=g) / math.sqrt(F)).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if E > 4:
        ids[ids == 1] = 2 if top == 1 else ids[ids == 1]    # with one choice per token: an expert that nobody chose
    weights = torch.rand(T, top, generator=g)
    shared = torch.randn(T, D, generator=g)
    zs = torch.randn(T, generator=g)
    x0 = torch.randn(T, D, generator=g)
    rows, group_off, tile_off = ops.group_rows(ids.to(DEV).view(-1), E)
    counts = torch.bincount(ids.view(-1).long(), minlength=E)
    assert group_off.cpu().tolist() == [0] + counts.cumsum(0).tolist()
    assert tile_off.cpu().tolist() == [0] + ((counts + 63) // 64).cumsum(0).tolist()
    listed = rows.cpu().long()
    assert sorted(listed.tolist()) == list(range(T * top))
    assert (ids.view(-1)[listed] == torch.repeat_interleave(torch.arange(E), counts).to(torch.int32)).all()
    u = torch.empty(T * top, F, dtype=torch.bfloat16, device=DEV)
    ops.grouped_gemm(h.to(DEV), w_up.to(DEV), u, listed=(rows, group_off, tile_off), a_div=top, act="gelu")
    pre = torch.einsum("tjfd,td->tjf", w_up.double()[ids.long()], h.double())
    assert _rel(u.reshape(T, top, F), 0.5 * pre * (1 + torch.erf(pre / math.sqrt(2.0)))) < 4e-3
    y = torch.empty(T * top, D, dtype=torch.float32, device=DEV)
    ops.grouped_gemm(u, w_down.to(DEV), y, listed=(rows, group_off, tile_off))
    y_ref = torch.einsum("tjdf,tjf->tjd", w_down.double()[ids.long()], u.double().cpu().reshape(T, top, F))
    assert _rel(y.reshape(T, top, D), y_ref) < 2e-6
    x = x0.clone().to(DEV)
    ops.moe_combine(y, weights.to(DEV), x, True, shared.to(DEV), zs.to(DEV))
    ref = x0.double() + (weights.double()[:, :, None] * y_ref).sum(1) + torch.sigmoid(zs.double())[:, None] * shared.double()
    assert _rel(x, ref) < 2e-6
    # the streaming kernels make the same rows
    u2 = ops.moe_up(h.to(DEV), w_up.to(DEV), ids.to(DEV), "gelu")
    assert _rel(u2, u.reshape(T, top, F)) < 4e-3


@pytest.mark.parametrize("T,E,top,D,F", [(300, 6, 1, 128, 48), (700, 16, 3, 104, 56), (512, 64, 6, 256, 320), (130, 3, 3, 64, 24)])
def test_the_experts_products_on_tcgen05_in_the_padded_order(T, E, top, D, F):
    """Every expert's pairs padded to whole tiles of 128 rows, both products as one tcgen05 launch each whose row tiles
    pick their expert's weight, tiles behind the last left out (their rows stay as they were: NaN here)."""
    ops = _ops()
    g = torch.Generator().manual_seed(T + E)
    h = torch.randn(T, D, generator=g).to(torch.bfloat16)
    w_up = (torch.randn(E, F, D, generator=g) / math.sqrt(D)).to(torch.bfloat16)
    w_down = (torch.randn(E, D, F, generator=g) / math.sqrt(F)).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if top == 1:
        ids[ids == 1] = 2                                   # an expert that nobody chose
    weights = torch.rand(T, top, generator=g)
    src, dst, tile_group = ops.group_rows_padded(ids.to(DEV).view(-1), E)
    src_h, dst_h, tg = src.cpu().long(), dst.cpu().long(), tile_group.cpu().tolist()
    flat = ids.view(-1).long()
    assert (src_h[dst_h] == torch.arange(T * top)).all() and int((src_h >= 0).sum()) == T * top
    for tile, grp in enumerate(tg):
        inside = src_h[tile * 128:(tile + 1) * 128]
        assert (grp == -1 and (inside < 0).all()) or (flat[inside[inside >= 0]] == grp).all()
    a = ops.gather_rows(h.to(DEV), src, top)
    assert (a.cpu()[dst_h].double() == h.double()[torch.arange(T * top) // top]).all() and float(a.cpu()[src_h < 0].abs().max()) == 0.0
    u = ops.gemm_tc_grouped(a, w_up.to(DEV), tile_group, torch.bfloat16)
    ops.activation(u, "gelu", out=u)
    pre = torch.einsum("tjfd,td->tjf", w_up.double()[ids.long()], h.double())
    got_u = u.cpu()[dst_h].reshape(T, top, F)
    assert _rel(got_u, 0.5 * pre * (1 + torch.erf(pre / math.sqrt(2.0)))) < 6e-3
    y = ops.gemm_tc_grouped(u, w_down.to(DEV), tile_group, torch.float32)
    y_ref = torch.einsum("tjdf,tjf->tjd", w_down.double()[ids.long()], got_u.double())
    assert _rel(y.cpu()[dst_h].reshape(T, top, D), y_ref) < 2e-5
    x = torch.zeros(T, D, device=DEV)
    ops.moe_combine(y, weights.to(DEV), x, False, place=dst)
    assert _rel(x, (weights.double()[:, :, None] * y_ref).sum(1)) < 2e-5
    ops.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dv", [(1, 600), (2, 512), (1, 2048), (1, 48)])
def test_all_heads_normed_together_with_weight_and_gate(dtype, H, dv):
    """The scan's raw outputs over the root mean square of a whole row (all heads as one head, or long heads), times a
    weight, times the gate's sigmoid: the form for heads of 512 values and more (a block per row) and the narrow one."""
    ops = _ops()
    g = torch.Generator().manual_seed(dv)
    rows = 9
    raw = 3.0 * torch.randn(rows, H, dv, generator=g)
    weight = 1 + 0.3 * torch.randn(H * dv, generator=g)
    gate = torch.randn(rows, H * dv + 7, generator=g).to(dtype)
    out = ops.head_norm_gate(raw.to(DEV), dv, 1e-5, dtype, weight=weight.to(DEV), gate=gate.to(DEV)[:, 3:3 + H * dv], act="sigmoid")
    x = raw.double()
    ref = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * weight.double().reshape(H, dv)
    ref = ref.reshape(rows, H * dv) * torch.sigmoid(gate.double()[:, 3:3 + H * dv])
    assert _rel(out, ref) < (2e-6 if dtype == torch.float32 else 4e-3)
