"""The kernels that the Fetorax design added, each alone against a plain float64 restatement, at sizes
and with inputs made so that a fault shows: a far key whose score stands out, a sink that takes most of the
weight, keys at page borders, values of another size than keys, states carried between calls, decays near one."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from longbow_quarrel_b200.kernels import ops
    return ops


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ attention: sink, gate, value size, far keys, page borders

def _paged(keys, values, page_size, seed):
    """Scatter [n, G, size] keys and values of one sequence into pools whose pages lie in a shuffled order."""
    n, G, hd = keys.shape
    vd = values.shape[2]
    n_pages = -(-n // page_size) + 3
    order = np.random.default_rng(seed).permutation(n_pages)
    k_pages = torch.full((n_pages, G, page_size, hd), float("nan"), dtype=keys.dtype, device=DEV)
    v_pages = torch.full((n_pages, G, page_size, vd), float("nan"), dtype=keys.dtype, device=DEV)
    table = np.full((2, n_pages), -1, dtype=np.int32)
    for p in range(-(-n // page_size)):
        table[1, p] = order[p]
        lo, hi = p * page_size, min(n, (p + 1) * page_size)
        k_pages[order[p], :, :hi - lo] = keys[lo:hi].transpose(0, 1)
        v_pages[order[p], :, :hi - lo] = values[lo:hi].transpose(0, 1)
    return k_pages, v_pages, _i32(table)


def _attention_plain64(q, keys, values, pos, scale, sink, gate):
    """q [H, hd] at position pos over keys[:pos + 1]; float64."""
    H, G = q.shape[0], keys.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (keys[:pos + 1, g].double() @ q[h].double()) * scale
        top = max(float(s.max()), float(sink[h])) if sink is not None else float(s.max())
        e = torch.exp(s - top)
        den = e.sum() + (np.exp(float(sink[h]) - top) if sink is not None else 0.0)
        o = (e[:, None] * values[:pos + 1, g].double()).sum(0) / den
        if gate is not None:
            o = o * torch.sigmoid(gate[h].double())
        out.append(o)
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,vd", [(6, 2, 32, 16), (1, 1, 24, 40), (4, 4, 64, 64), (3, 1, 130, 200)])
def test_attention_with_a_sink_a_gate_and_a_key_that_stands_out(dtype, H, G, hd, vd):
    ops = _ops()
    gen = torch.Generator().manual_seed(H * 100 + hd)
    n, page = 300, 64
    keys = (0.3 * torch.randn(n, G, hd, generator=gen)).to(dtype)
    values = torch.randn(n, G, vd, generator=gen).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    # The key that must be found: at the first position, on both sides of page borders, far back, and the token's own.
    for star in (0, 63, 64, 65, 127, 128, 299):
        k2 = keys.clone()
        k2[star, :, 0] = 12.0                                   # this key's score stands out for queries along dimension 0
        k_pages, v_pages, table = _paged(k2.to(DEV), values.to(DEV), page, seed=star)
        for pos in sorted({star, min(star + 1, n - 1), n - 1}):
            q = (0.3 * torch.randn(2, H * hd + 7, generator=gen)).to(dtype)          # rows wider than q: a strided buffer
            q[:, 0:H * hd:hd] = 8.0
            gate = torch.randn(2, H * vd, generator=gen).to(dtype)
            sink = torch.linspace(25.0, -2.0, H)                  # the first head's sink outweighs even that key
            for use_sink, use_gate in ((True, True), (False, False), (True, False)):
                got = ops.attention_plain(q.to(DEV), k_pages, v_pages, table, _i32([pos, pos]), _i32([0, 1]), _i32([1, 1]),
                                          H, G, hd, page, 0.2, None, vd=vd, sink=sink.to(DEV) if use_sink else None,
                                          gate=gate.to(DEV) if use_gate else None).float().cpu()
                for row in range(2):
                    ref = _attention_plain64(q[row, :H * hd].reshape(H, hd), k2, values, pos, 0.2, sink if use_sink else None,
                                             gate[row].reshape(H, vd) if use_gate else None).reshape(-1)
                    err = float((got[row].double() - ref).abs().max() / ref.abs().max().clamp_min(1e-6))
                    assert err < tol, (star, pos, use_sink, use_gate, err)
                    if not use_sink and not use_gate and pos >= star:
                        # Without a sink nearly all weight lies on the one key: the output is its value.
                        want = values[star, torch.arange(H) // (H // G)].reshape(-1).double()
                        assert float((ref - want).abs().max()) < 0.05 * float(want.abs().max())


# ------------------------------------------------------------------ biases, partial rotation and the cache write

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,vd,rot", [(4, 2, 16, 24, 8), (2, 1, 32, 32, 32), (3, 3, 20, 6, 0), (1, 1, 64, 64, 2)])
def test_biases_partial_rotation_and_cache_write(dtype, H, G, hd, vd, rot):
    ops = _ops()
    gen = torch.Generator().manual_seed(hd + rot)
    T, page, n_pos = 5, 64, 200
    width = (H + G) * hd + G * vd + 11
    buf = torch.randn(T, width, generator=gen).to(dtype)
    bias = torch.randn(width, generator=gen)
    pos = [0, 63, 64, 130, 199]
    f = 100.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1)) / 3.0
    ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * f[None, :]
    cos, sin = torch.cos(ang).float().contiguous(), torch.sin(ang).float().contiguous()
    k_pages = torch.zeros(4, G, page, hd, dtype=dtype, device=DEV)
    v_pages = torch.zeros(4, G, page, vd, dtype=dtype, device=DEV)
    table = _i32([[3, 0, 2, 1]])
    dev = buf.to(DEV)
    ops.rope_partial(dev, bias.to(DEV), cos.to(DEV) if rot else None, sin.to(DEV) if rot else None, rot, _i32(pos), _i32([0] * T),
                     _i32([0]), table, k_pages, v_pages, H + G, H, G, hd, vd, (H + G) * hd, page)
    got = dev.float().cpu().double()
    x = buf.double() + bias.double()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    pages = [3, 0, 2, 1]
    for t in range(T):
        for head in range(H + G):
            v = x[t, head * hd:(head + 1) * hd].clone()
            u, w = v[:rot // 2].clone(), v[rot // 2:rot].clone()
            c, s = cos[pos[t]].double(), sin[pos[t]].double()
            v[:rot // 2], v[rot // 2:rot] = u * c - w * s, w * c + u * s
            if head < H:            # queries come back in place; keys go to the cache only
                assert float((got[t, head * hd:(head + 1) * hd] - v).abs().max()) < tol * max(1.0, float(v.abs().max()))
            if head >= H:
                stored = k_pages[pages[pos[t] // page], head - H, pos[t] % page].float().cpu().double()
                assert float((stored - v).abs().max()) < tol * max(1.0, float(v.abs().max()))
        for g in range(G):
            v = x[t, (H + G) * hd + g * vd:(H + G) * hd + (g + 1) * vd]
            stored = v_pages[pages[pos[t] // page], g, pos[t] % page].float().cpu().double()
            assert float((stored - v).abs().max()) < tol * max(1.0, float(v.abs().max()))
    # Columns beyond the values (a gate's, say) are left alone.
    assert torch.equal(dev[:, (H + G) * hd + G * vd:].cpu(), buf[:, (H + G) * hd + G * vd:])
    if dtype == torch.bfloat16:
        # Float32 rows in, bfloat16 queries and cache out: rounded once, after bias and rotation; the rows stay as they were.
        wide = buf.float().to(DEV)
        q16 = torch.zeros(T, H * hd, dtype=dtype, device=DEV)
        k2, v2 = torch.zeros_like(k_pages), torch.zeros_like(v_pages)
        ops.rope_partial(wide, bias.to(DEV), cos.to(DEV) if rot else None, sin.to(DEV) if rot else None, rot, _i32(pos),
                         _i32([0] * T), _i32([0]), table, k2, v2, H + G, H, G, hd, vd, (H + G) * hd, page, qout=q16)
        assert torch.equal(wide.cpu(), buf.float())
        assert float((q16.float().cpu().double() - got[:, :H * hd]).abs().max()) < 2 * tol * float(got.abs().max())
        assert float((k2.float() - k_pages.float()).abs().max()) < 2 * tol * float(got.abs().max())
        assert float((v2.float() - v_pages.float()).abs().max()) < 2 * tol * float(got.abs().max())


# ------------------------------------------------------------------ the recurrent scan

def _scan64(q, k, v, a, b):
    """o_t = S_t^T q_t with S_t = a_t S + b_t k_t v_t^T; all [T, ...] float64, one head."""
    S = torch.zeros(k.shape[1], v.shape[1], dtype=torch.float64)
    out = []
    for t in range(q.shape[0]):
        S = a[t] * S + b[t] * torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out), S


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv,rot", [(2, 16, 24, 8), (1, 72, 5, 0), (3, 136, 33, 136), (2, 64, 64, 32), (1, 256, 17, 0)])
def test_retention_scan_in_pieces_and_batches(dtype, H, dk, dv, rot):
    """Three sequences of unequal lengths in shuffled slots, their tokens given in two calls (the state is carried
    in the slot); decays from 0.5 to one exactly, so that the first token's trace must survive to the last."""
    ops = _ops()
    gen = torch.Generator().manual_seed(dk + dv)
    lens, cut = [150, 1, 37], [100, 0, 2]
    decay = torch.linspace(0.5, 1.0, H)
    width = H * (2 * dk + dv) + 3
    n_pos = 160
    f = 1000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))
    ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * f[None, :]
    cos, sin = torch.cos(ang).float().contiguous().to(DEV), torch.sin(ang).float().contiguous().to(DEV)
    rows = [torch.randn(n, width, generator=gen).to(dtype) for n in lens]
    for r in rows:
        r[0, 2 * H * dk:2 * H * dk + H * dv] *= 20.0            # the first token's values are large: they must last
    slots = [5, 0, 3]
    state = torch.full((7, H, dk, dv), float("nan"), device=DEV)
    state[slots] = 0.0
    got = [[] for _ in lens]
    for part in range(2):
        live = [i for i in range(3) if (cut[i] if part == 0 else lens[i] - cut[i]) > 0]
        pieces = [rows[i][:cut[i]] if part == 0 else rows[i][cut[i]:] for i in live]
        cu = np.concatenate([[0], np.cumsum([len(p) for p in pieces])])
        pos = np.concatenate([np.arange(len(p)) + (0 if part == 0 else cut[i]) for i, p in zip(live, pieces)])
        raw, _ = ops.linear_scan(torch.cat(pieces).to(DEV), 0, H * dk, 2 * H * dk, state, _i32(cu), _i32([slots[i] for i in live]),
                                 _i32(pos), len(live), H, dk, dv, k_scale=dk ** -0.5, decay=decay.to(DEV),
                                 rot=(cos, sin, rot) if rot else None)
        for n, i in enumerate(live):
            got[i].append(raw[cu[n]:cu[n + 1]].cpu().double())
    tol = 2e-5
    for i, n in enumerate(lens):
        x = rows[i].double()
        for h in range(H):
            q, k = x[:, h * dk:(h + 1) * dk].clone(), x[:, (H + h) * dk:(H + h + 1) * dk].clone()
            if rot:
                c, s = torch.cos(ang[:n]), torch.sin(ang[:n])
                for z in (q, k):
                    u, w = z[:, :rot // 2].clone(), z[:, rot // 2:rot].clone()
                    z[:, :rot // 2], z[:, rot // 2:rot] = u * c - w * s, w * c + u * s
            v = x[:, 2 * H * dk + h * dv:2 * H * dk + (h + 1) * dv]
            ref, S = _scan64(q, k * dk ** -0.5, v, [float(decay[h])] * n, [1.0] * n)
            mine = torch.cat(got[i])[:, h]
            assert float((mine - ref).abs().max()) < tol * float(ref.abs().max()), (i, h)
            assert float((state[slots[i], h].cpu().double() - S).abs().max()) < tol * float(S.abs().max())
    assert torch.isnan(state[[1, 2, 4, 6]]).all()             # other slots are not touched


@pytest.mark.parametrize("H,dk,dv,cap", [(2, 8, 16, 5.0), (1, 72, 20, 15.0), (3, 24, 40, 8.0), (2, 64, 64, 10.0)])
def test_gated_scan_follows_the_stabilised_recurrence(H, dk, dv, cap):
    """The gates in their extremes as well: pre-activations far beyond the cap on both sides, so that the running
    maximum moves up and down, and a forget gate that is nearly shut."""
    ops = _ops()
    gen = torch.Generator().manual_seed(dk * dv)
    lens = [90, 3]
    width = H * (2 * dk + dv)
    rows = [torch.randn(n, width, generator=gen) for n in lens]
    pre = [torch.randn(n, 2 * H, generator=gen) * 3 * cap for n in lens]
    pre[0][40:50, H:] = -4 * cap                                  # forget nearly everything for ten tokens
    bias = torch.randn(2 * H, generator=gen)
    state = torch.zeros(4, H, dk + 1, dv + 1, device=DEV)
    got_raw, got_enm = [], []
    # the first sequence in two calls, the second alone in between
    for piece, pg, slot, at in ((rows[0][:33], pre[0][:33], 2, 0), (rows[1], pre[1], 0, 0), (rows[0][33:], pre[0][33:], 2, 33)):
        n = len(piece)
        raw, enm = ops.linear_scan(piece.to(DEV), 0, H * dk, 2 * H * dk, state, _i32([0, n]), _i32([slot]), _i32(list(range(at, at + n))),
                                   1, H, dk, dv, q_scale=dk ** -0.5, gates=(pg.contiguous().to(DEV), bias.to(DEV), cap))
        got_raw.append(raw.cpu().double())
        got_enm.append(enm.cpu().double())
    mine = {0: (torch.cat([got_raw[0], got_raw[2]]), torch.cat([got_enm[0], got_enm[2]])), 1: (got_raw[1], got_enm[1])}
    for i, n in enumerate(lens):
        x, g = rows[i].double(), pre[i].double() + bias.double()
        for h in range(H):
            li = cap * torch.tanh(g[:, h] / cap)
            lf = torch.nn.functional.logsigmoid(cap * torch.tanh(g[:, H + h] / cap))
            m, a, b, ms = 0.0, [], [], []
            for t in range(n):
                m_new = max(float(lf[t]) + m, float(li[t]))
                a.append(np.exp(float(lf[t]) + m - m_new))
                b.append(np.exp(float(li[t]) - m_new))
                m = m_new
                ms.append(m)
            q = x[:, h * dk:(h + 1) * dk] * dk ** -0.5
            k = x[:, (H + h) * dk:(H + h + 1) * dk]
            v = torch.cat([x[:, 2 * H * dk + h * dv:2 * H * dk + (h + 1) * dv], torch.ones(n, 1, dtype=torch.float64)], dim=1)
            ref, _ = _scan64(q, k, v, a, b)
            raw, enm = mine[i]
            assert float((raw[:, h] - ref).abs().max()) < 3e-5 * float(ref.abs().max()), (i, h)
            assert float((enm[:, h] - torch.exp(-torch.tensor(ms))).abs().max()) < 1e-5 * float(np.exp(-min(ms)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unit_norm_per_head_with_weight_denominator_and_gate(dtype):
    ops = _ops()
    gen = torch.Generator().manual_seed(9)
    rows, H, dv = 7, 3, 20
    raw = torch.randn(rows, H, dv + 1, generator=gen) * 5
    raw[0] *= 1e-4                                              # tiny outputs: epsilon matters
    enm = torch.rand(rows, H, generator=gen) * 3
    weight = torch.randn(H * dv, generator=gen)
    gate = torch.randn(rows, H * dv + 5, generator=gen).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for act, fn in (("sigmoid", torch.sigmoid), ("silu", torch.nn.functional.silu), (None, None)):
        for with_den in (True, False):
            got = ops.head_norm_gate((raw if with_den else raw[..., :dv].contiguous()).to(DEV), dv, 1e-5, dtype,
                                     exp_neg_m=enm.to(DEV) if with_den else None, weight=weight.to(DEV),
                                     gate=gate.to(DEV)[:, 2:2 + H * dv] if act else None, act=act).float().cpu().double()
            o = raw[..., :dv].double()
            if with_den:
                o = o / (torch.maximum(raw[..., dv].double().abs(), enm.double()) + 1e-6)[..., None]
            o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5)
            o = o.reshape(rows, H * dv) * weight.double()
            if act:
                o = o * fn(gate[:, 2:2 + H * dv].double())
            assert float((got - o).abs().max()) < tol * float(o.abs().max()), (act, with_den)


# ------------------------------------------------------------------ the small pieces

@pytest.mark.parametrize("D", [48, 100, 1024, 4100])
def test_a_normed_branch_joins_the_stream_and_the_next_norm_comes_with_it(D):
    ops = _ops()
    gen = torch.Generator().manual_seed(D)
    y, x = torch.randn(5, D, generator=gen) * 7, torch.randn(5, D, generator=gen)
    g1, g2 = 1 + 0.2 * torch.randn(D, generator=gen), 1 + 0.2 * torch.randn(D, generator=gen)
    want_x = x.double() + y.double() / torch.sqrt((y.double() ** 2).mean(-1, keepdim=True) + 1e-6) * g1.double()
    want_h = want_x / torch.sqrt((want_x ** 2).mean(-1, keepdim=True) + 1e-5) * g2.double()
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        xd = x.clone().to(DEV)
        h = ops.rmsnorm_add(y.to(DEV), g1.to(DEV), 1e-6, xd, (g2.to(DEV), 1e-5), dtype)
        assert float((xd.cpu().double() - want_x).abs().max()) < 1e-5 * float(want_x.abs().max())
        assert float((h.float().cpu().double() - want_h).abs().max()) < tol * float(want_h.abs().max())
        xd = x.clone().to(DEV)
        assert ops.rmsnorm_add(y.to(DEV), g1.to(DEV), 1e-6, xd) is None
        assert float((xd.cpu().double() - want_x).abs().max()) < 1e-5 * float(want_x.abs().max())


def test_activations_and_soft_cap():
    ops = _ops()
    x = torch.linspace(-6, 6, 1001)
    ref = {"relu2": torch.relu(x.double()) ** 2, "silu": torch.nn.functional.silu(x.double()), "relu": torch.relu(x.double()),
           "gelu_tanh": torch.nn.functional.gelu(x.double(), approximate="tanh")}
    for kind, want in ref.items():
        got = ops.activation(x.to(DEV), kind).cpu().double()
        assert float((got - want).abs().max()) < 1e-5, kind
        got = ops.activation(x.to(torch.bfloat16).to(DEV), kind).float().cpu().double()
        want16 = {"relu2": lambda z: torch.relu(z) ** 2, "silu": torch.nn.functional.silu, "relu": torch.relu,
                  "gelu_tanh": lambda z: torch.nn.functional.gelu(z, approximate="tanh")}[kind](x.to(torch.bfloat16).double())
        assert float((got - want16).abs().max()) < 0.3, kind
        assert float(((got - want16).abs() / want16.abs().clamp_min(1.0)).max()) < 5e-3, kind
    z = torch.linspace(-200, 200, 777).reshape(7, 111).contiguous()
    got = ops.softcap(z.clone().to(DEV), 30.0).cpu().double()
    assert float((got - 30.0 * torch.tanh(z.double() / 30.0)).abs().max()) < 1e-4


@pytest.mark.parametrize("rows,N,K", [(1, 2, 48), (9, 6, 100), (300, 64, 2048), (5, 8, 4100)])
def test_a_projection_onto_few_outputs_in_32_bit(rows, N, K):
    ops = _ops()
    gen = torch.Generator().manual_seed(K)
    x, w = torch.randn(rows, K, generator=gen), torch.randn(N, K, generator=gen)
    for xt, wt in ((torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16)):
        xs, ws = x.to(xt), w.to(wt)
        got = ops.small_proj(xs.to(DEV), ws.to(DEV)).cpu().double()
        want = xs.double() @ ws.double().T
        assert float((got - want).abs().max()) < 2e-6 * K ** 0.5 * float(want.abs().max())
    # a row's result does not depend on the rows beside it
    alone = ops.small_proj(x[:1].contiguous().to(DEV), w.to(DEV))
    assert torch.equal(alone[0], ops.small_proj(x.to(DEV), w.to(DEV))[0])


@pytest.mark.parametrize("mlstm", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv,rot", [(2, 16, 24, 8), (1, 72, 5, 0), (3, 136, 33, 136), (2, 64, 64, 32), (1, 256, 70, 2)])
def test_the_single_token_form_of_the_scan_agrees_with_the_chunked_one(H, dk, dv, rot, mlstm, dtype):
    """Five sequences in shuffled slots with states left by prompts of unequal lengths; then one token each through
    the kernel for prompts and through the one for single tokens: the same outputs and the same states."""
    ops = _ops()
    gen = torch.Generator().manual_seed(dk + dv + int(mlstm))
    B, lens, slots = 5, [40, 1, 17, 64, 3], [6, 0, 3, 1, 4]
    width = H * (2 * dk + dv) + 5
    cos = torch.rand(80, max(rot // 2, 1), generator=gen).to(DEV).contiguous()
    sin = torch.rand(80, max(rot // 2, 1), generator=gen).to(DEV).contiguous()
    decay = torch.linspace(0.9, 0.999, H).to(DEV)
    bias = torch.randn(2 * H, generator=gen).to(DEV)

    def call(rows, state, cu, pos, n_seq, single):
        kw = dict(gates=(torch.randn(rows.shape[0], 2 * H, generator=torch.Generator().manual_seed(rows.shape[0])).mul(4.0).to(DEV),
                         bias, 6.0), q_scale=dk ** -0.5) if mlstm else \
            dict(decay=decay, k_scale=dk ** -0.5, rot=(cos[:, :rot // 2].contiguous(), sin[:, :rot // 2].contiguous(), rot) if rot else None)
        return ops.linear_scan(rows.to(DEV), 3, 3 + H * dk, 3 + 2 * H * dk, state, _i32(cu), _i32(slots[:n_seq]), _i32(pos), n_seq,
                               H, dk, dv, single=single, **kw)

    state = torch.zeros(8, H, dk + int(mlstm), dv + int(mlstm), device=DEV)
    prompt = torch.randn(sum(lens), width, generator=gen).to(dtype)
    cu = np.concatenate([[0], np.cumsum(lens)])
    call(prompt, state, cu, np.concatenate([np.arange(n) for n in lens]), B, False)
    step = torch.randn(B, width, generator=gen).to(dtype)
    s_chunked, s_single = state.clone(), state.clone()
    raw_c, enm_c = call(step, s_chunked, np.arange(B + 1), lens, B, False)
    raw_s, enm_s = call(step, s_single, np.arange(B + 1), lens, B, True)
    scale = float(raw_c.abs().max())
    assert float((raw_s - raw_c).abs().max()) < 1e-5 * scale
    assert float((s_single - s_chunked).abs().max()) < 1e-5 * float(s_chunked.abs().max())
    if mlstm:
        assert float((enm_s - enm_c).abs().max()) < 1e-5 * float(enm_c.abs().max())
    untouched = [i for i in range(8) if i not in slots]
    assert float(s_single[untouched].abs().max()) == 0.0
