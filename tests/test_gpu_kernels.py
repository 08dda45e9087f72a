"""Each kernel alone against a plain float32 torch restatement, at sizes other
than the engine's tiny models: widths and vocabularies that are no power of
two, head sizes in steps of 16, odd token counts, page edges."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


def K():
    from prelude_b200.ops import kernels
    return kernels


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("T,H,V", [(1, 64, 100), (37, 2560, 1000), (5, 100, 331)])
def test_embed_gather(dtype, T, H, V):
    table = rnd(V, H, dtype=dtype)
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    ids[0] = V - 1
    out = K().embed_gather(ids, table)
    assert out.dtype == torch.float32 and torch.equal(out, table.float()[ids.long()])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("T,H", [(1, 64), (19, 2560), (3, 100), (2, 8192), (4, 9000), (7, 72), (32, 5120), (1, 1024),
                                 (33, 4096), (8, 1100)])
@pytest.mark.parametrize("eps", [1e-6, 1e-3])
def test_add_rmsnorm(dtype, T, H, eps):
    x, res, w = rnd(T, H, dtype=dtype, seed=1), rnd(T, H, seed=2), 1 + 0.3 * rnd(H, seed=3)
    want_res = res + x.float()
    want = want_res / torch.sqrt((want_res * want_res).mean(-1, keepdim=True) + eps) * w
    res2 = res.clone()
    y = K().add_rmsnorm(x, res2, w, eps, dtype)
    assert torch.allclose(res2, want_res, atol=1e-6)            # the sum is kept in 32-bit
    assert (y.float() - want).abs().max() <= tol(dtype, float(want.abs().max()))
    # without the add the residual is left alone
    res3 = res.clone()
    y0 = K().add_rmsnorm(None, res3, w, eps, dtype)
    want0 = res / torch.sqrt((res * res).mean(-1, keepdim=True) + eps) * w
    assert torch.equal(res3, res) and (y0.float() - want0).abs().max() <= tol(dtype, float(want0.abs().max()))
    # chosen rows only
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
    yg = K().gather_add_rmsnorm(x, res, rows, w, eps, dtype)
    assert torch.equal(res, res3) and (yg.float() - want[rows.long()]).abs().max() <= tol(dtype, float(want.abs().max()))
    # plain norm of a tensor of the run's type
    yn = K().rmsnorm(x, w, eps)
    xf = x.float()
    wantn = xf / torch.sqrt((xf * xf).mean(-1, keepdim=True) + eps) * w
    assert (yn.float() - wantn).abs().max() <= tol(dtype, float(wantn.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("T,H,parts", [(8, 2560, 4), (3, 100, 2), (1, 64, 1), (5, 9000, 3), (7, 74, 5), (16, 4096, 2),
                                       (1, 5120, 6)])
def test_add_rmsnorm_of_partial_sums(dtype, T, H, parts):
    # the addend as float32 parts to be added up (a product whose K was cut): same result as adding their sum
    from prelude_b200.ops.kernels import PartialSums
    eps = 1e-5
    p, res, w = rnd(parts, T, H, seed=4), rnd(T, H, seed=2), 1 + 0.3 * rnd(H, seed=3)
    total = res.clone()
    for i in range(parts):
        total += p[i]
    want = total / torch.sqrt((total * total).mean(-1, keepdim=True) + eps) * w
    res2 = res.clone()
    y = K().add_rmsnorm(PartialSums(p), res2, w, eps, dtype)
    assert torch.equal(res2, total)                             # the parts in ascending order, in 32-bit
    assert (y.float() - want).abs().max() <= tol(dtype, float(want.abs().max()))
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
    yg = K().gather_add_rmsnorm(PartialSums(p), res, rows, w, eps, dtype)
    assert (yg.float() - want[rows.long()]).abs().max() <= tol(dtype, float(want.abs().max()))
    assert (PartialSums(p).materialize(torch.float32) - p.sum(0)).abs().max() == 0
    with pytest.raises(Exception, match="against residual"):
        K().add_rmsnorm(PartialSums(rnd(2, T, H + 4)), res2, w, eps, dtype)


@pytest.mark.parametrize("splits", [2, 4])
@pytest.mark.parametrize("M,N,K_", [(8, 2560, 9728), (3, 100, 8192), (16, 300, 4096)])
def test_gemm_stream_partial_sums(M, N, K_, splits):
    from prelude_b200.ops.linear import gemm_stream, linear, stream_splits
    from prelude_b200.ops.kernels import PartialSums
    x, w = rnd(M, K_, dtype=torch.bfloat16, seed=21), rnd(N, K_, dtype=torch.bfloat16, seed=22, scale=0.05)
    want = x.double() @ w.double().T
    parts = gemm_stream(x, w, splits=splits)
    assert parts.shape == (splits, M, N) and parts.dtype == torch.float32
    assert (parts.double().sum(0) - want).abs().max() <= 2e-3 * max(1.0, float(want.abs().max()))
    # every part is the product over its own columns
    kp = K_ // splits
    for s in range(splits):
        wp = x[:, s * kp:(s + 1) * kp].double() @ w[:, s * kp:(s + 1) * kp].double().T
        assert (parts[s].double() - wp).abs().max() <= 2e-3 * max(1.0, float(wp.abs().max()))
    got = linear(x, w, partial_sums_ok=True)
    if stream_splits(M, N, K_) > 1:
        assert isinstance(got, PartialSums) and got.parts.shape[0] == stream_splits(M, N, K_)
    else:
        assert isinstance(got, torch.Tensor)
    assert isinstance(linear(x, w), torch.Tensor)               # never unless the caller says its reader can take them


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("T,I", [(1, 8), (13, 9728), (6, 200), (3, 37), (2050, 1216), (5, 48)])
def test_silu_mul(dtype, T, I):
    gu = rnd(T, 2 * I, dtype=dtype, scale=3.0)
    g, u = gu.float()[:, :I], gu.float()[:, I:]
    want = g / (1 + torch.exp(-g)) * u
    got = K().silu_mul(gu)
    assert (got.float() - want).abs().max() <= tol(dtype, float(want.abs().max()))
    # gates far out on both sides: silu(g) -> 0 and -> g, never a NaN or an infinity
    far = torch.tensor([-300.0, -100.0, -88.0, -20.0, 0.0, 20.0, 88.0, 300.0], device=DEV)[:I]
    gu2 = gu.clone()
    gu2[0, :far.numel()] = far.to(dtype)
    gu2[0, I:I + far.numel()] = 2.0
    got2 = K().silu_mul(gu2).float()
    g2 = gu2.float()[0, :far.numel()]
    want2 = g2 / (1 + torch.exp(-g2)) * 2.0
    assert torch.isfinite(got2).all() and (got2[0, :far.numel()] - want2).abs().max() <= tol(dtype, 600.0)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (33, 100, 72), (130, 331, 200), (2, 2560, 9728), (65, 64, 16)])
def test_gemm_ref(dtype, M, N, K_):
    a, w, b = rnd(M, K_, dtype=dtype, seed=4), rnd(N, K_, dtype=dtype, seed=5), rnd(N, seed=6)
    want = a.double() @ w.double().T
    got = K().gemm_ref(a, w)
    scale = float(want.abs().max())
    assert (got.double() - want).abs().max() <= tol(dtype, scale) * (1 if dtype == torch.bfloat16 else 4)
    got_b = K().gemm_ref(a, w, b, torch.float32)
    assert got_b.dtype == torch.float32 and (got_b.double() - (want + b.double())).abs().max() <= 1e-5 * scale * 4
    # rows do not depend on what else is in the batch
    if M > 2:
        assert torch.equal(K().gemm_ref(a[1:2].contiguous(), w), got[1:2])
    # strided input rows (a view into a wider tensor)
    wide = rnd(M, K_ + 24, dtype=dtype, seed=7)
    assert torch.equal(K().gemm_ref(wide[:, 8:8 + K_], w), K().gemm_ref(wide[:, 8:8 + K_].contiguous(), w))


def _stored(rows, dtype):
    """A run of token rows [..., page_size, D] as the page layout stores it: for bfloat16
    pages with D % 64 == 0 the 16-byte chunks of token r are permuted, chunk c sits at c ^ (r & 7)."""
    D, ps = rows.shape[-1], rows.shape[-2]
    if not (dtype == torch.bfloat16 and D % 64 == 0):
        return rows
    chunks = rows.reshape(*rows.shape[:-1], D // 8, 8)
    out = torch.empty_like(chunks)
    for r in range(ps):
        for c in range(D // 8):
            out[..., r, c ^ (r & 7), :] = chunks[..., r, c, :]
    return out.reshape(rows.shape)


def _put(pages_tensor, page, in_page, row):
    """Write one token's [nKV, D] row into its page at the stored position of every chunk."""
    D = row.shape[-1]
    if pages_tensor.dtype == torch.bfloat16 and D % 64 == 0:
        ch = row.reshape(row.shape[0], D // 8, 8)
        perm = torch.tensor([c ^ (in_page & 7) for c in range(D // 8)])
        stored = torch.empty_like(ch)
        stored[:, perm] = ch
        pages_tensor[page, :, in_page] = stored.reshape(row.shape)
    else:
        pages_tensor[page, :, in_page] = row


def _get(pages_tensor, page, in_page):
    D = pages_tensor.shape[-1]
    row = pages_tensor[page, :, in_page]
    if pages_tensor.dtype == torch.bfloat16 and D % 64 == 0:
        ch = row.reshape(row.shape[0], D // 8, 8)
        perm = torch.tensor([c ^ (in_page & 7) for c in range(D // 8)])
        return ch[:, perm].reshape(row.shape)
    return row


def _paged(k, v, page_size, num_pages, seed):
    """Scatter dense [L, nKV, D] keys and values into randomly chosen pages."""
    L = k.shape[0]
    n = -(-L // page_size)
    g = torch.Generator().manual_seed(seed)
    pages = torch.randperm(num_pages, generator=g)[:n].tolist()
    kp = torch.full((num_pages, k.shape[1], page_size, k.shape[2]), float("nan"), dtype=k.dtype, device=DEV)
    vp = torch.full_like(kp, float("nan"))
    for i in range(L):
        _put(kp, pages[i // page_size], i % page_size, k[i])
        _put(vp, pages[i // page_size], i % page_size, v[i])
    return kp, vp, pages


def _attention_plain(q, k, v, pos_q, scale, window):
    """q [T, nH, D] at absolute positions pos_q against keys 0..L-1 (float64)."""
    nH, nKV = q.shape[1], k.shape[1]
    kx, vx = k.double().repeat_interleave(nH // nKV, 1), v.double().repeat_interleave(nH // nKV, 1)
    s = torch.einsum("ihd,jhd->hij", q.double(), kx) * scale
    j = torch.arange(k.shape[0], device=q.device)[None, :]
    i = torch.as_tensor(pos_q, device=q.device)[:, None]
    vis = j <= i
    if window:
        vis = vis & (i - j < window)
    s = s.masked_fill(~vis[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), vx)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nH,nKV,D,page", [(4, 2, 16, 4), (6, 2, 32, 8), (5, 1, 48, 16), (8, 8, 64, 16),
                                           (3, 3, 80, 16), (8, 2, 128, 16), (2, 1, 256, 32)])
@pytest.mark.parametrize("window", [None, 5, 37])
def test_paged_attention_ref(dtype, nH, nKV, D, page, window):
    L = 83
    k, v = rnd(L, nKV, D, dtype=dtype, seed=1), rnd(L, nKV, D, dtype=dtype, seed=2)
    kp, vp, pages = _paged(k, v, page, 40, seed=3)
    pos = [0, 1, page - 1, page, page + 1, 31, 32, 33, 63, 64, L - 1, 40, 41]      # page and block edges
    q = rnd(len(pos), nH, D, dtype=dtype, seed=4)
    table = torch.full((2, 24), -1, dtype=torch.int32, device=DEV)
    table[1, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
    got = K().paged_attention_ref(q, kp, vp, torch.tensor(pos, dtype=torch.int32, device=DEV),
                                  torch.ones(len(pos), dtype=torch.int32, device=DEV), table, 1 / math.sqrt(D), window)
    want = _attention_plain(q, k, v, pos, 1 / math.sqrt(D), window)
    assert not torch.isnan(got.float()).any()
    assert (got.double() - want).abs().max() <= tol(dtype, 4.0)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("where", ["far", "page_edge", "window_first", "just_outside_window", "self"])
def test_attention_finds_the_one_key_that_matters(dtype, where):
    """One key among hundreds is made to dominate; a kernel that skipped it, or
    read one past the window, would return another value row."""
    nH, nKV, D, page, L, window = 4, 2, 64, 16, 400, 100
    k, v = rnd(L, nKV, D, dtype=dtype, seed=1, scale=0.1), rnd(L, nKV, D, dtype=dtype, seed=2)
    q = rnd(1, nH, D, dtype=dtype, seed=3, scale=0.1)
    pos = L - 1
    target = {"far": 3, "page_edge": 15 * page, "window_first": pos - window + 1,
              "just_outside_window": pos - window, "self": pos}[where]
    unit = torch.zeros(D, device=DEV)
    unit[5] = 1.0
    q[0, :, :] = (unit * 40).to(dtype)
    k[target, :, :] = (unit * 40).to(dtype)                 # score 1600 * scale = 200 against ~0 elsewhere
    kp, vp, pages = _paged(k, v, page, 64, seed=5)
    table = torch.tensor([pages], dtype=torch.int32, device=DEV)
    use_window = window if where in ("window_first", "just_outside_window") else None
    got = K().paged_attention_ref(q, kp, vp, torch.tensor([pos], dtype=torch.int32, device=DEV),
                                  torch.zeros(1, dtype=torch.int32, device=DEV), table, 1 / math.sqrt(D), use_window)
    want = _attention_plain(q, k, v, [pos], 1 / math.sqrt(D), use_window)
    assert (got.double() - want).abs().max() <= tol(dtype, 4.0)
    hit = (got[0, 0].float() - v[target, 0].float()).abs().max() < 0.05
    assert hit == (where != "just_outside_window")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nH,nKV,D,rot", [(4, 2, 16, 16), (6, 2, 32, 32), (5, 1, 48, 48), (8, 2, 128, 128),
                                          (3, 3, 80, 32), (2, 1, 256, 256), (2, 2, 64, 0), (4, 2, 128, 64),
                                          (4, 4, 64, 32), (2, 1, 128, 24), (32, 8, 128, 128), (3, 1, 32, 16)])
@pytest.mark.parametrize("norm,interleaved", [(True, False), (False, False), (True, True)])
def test_qknorm_rope_kvwrite(dtype, nH, nKV, D, rot, norm, interleaved):
    # interleaved: angle j turns elements 2 j and 2 j + 1 instead of j and j + rot / 2
    T, page, num_pages, eps, theta = 11, 8, 9, 1e-5, 10000.0
    qkv = rnd(T, (nH + 2 * nKV) * D, dtype=dtype, seed=1)
    qw, kw = (1 + 0.2 * rnd(D, seed=2), 1 + 0.2 * rnd(D, seed=3)) if norm else (None, None)
    cos = sin = None
    if rot:
        inv = torch.tensor([1.0 / theta ** (i / rot) for i in range(0, rot, 2)], dtype=torch.float64).float()
        ang = torch.arange(64, dtype=torch.float32)[:, None] * inv[None]
        cos, sin = ang.cos().to(DEV), ang.sin().to(DEV)
    # two requests: rows 0..6 are positions 3..9 of request 1, rows 7..10 positions 0..3 of request 0
    positions = torch.tensor([3, 4, 5, 6, 7, 8, 9, 0, 1, 2, 3], dtype=torch.int32, device=DEV)
    seq = torch.tensor([1] * 7 + [0] * 4, dtype=torch.int32, device=DEV)
    table = torch.tensor([[4, -1], [7, 2]], dtype=torch.int32, device=DEV)
    kp = torch.zeros(num_pages, nKV, page, D, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_out = K().qknorm_rope_kvwrite(qkv, nH, nKV, D, qw, kw, eps, cos, sin, rot, positions, seq, table, kp, vp, True, status,
                                    interleaved=interleaved)
    assert int(status.item()) == 0

    def plain(x, w):
        x = x.float()
        if w is not None:
            x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w
        if rot:
            c, s = cos[positions.long()][:, None, :], sin[positions.long()][:, None, :]
            if interleaved:
                x1, x2, rest = x[..., 0:rot:2], x[..., 1:rot:2], x[..., rot:]
                turned = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], -1).reshape(*x.shape[:-1], rot)
                x = torch.cat([turned, rest], -1)
            else:
                x1, x2, rest = x[..., :rot // 2], x[..., rot // 2:rot], x[..., rot:]
                x = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], -1)
        return x
    q = qkv[:, :nH * D].reshape(T, nH, D)
    k = qkv[:, nH * D:(nH + nKV) * D].reshape(T, nKV, D)
    v = qkv[:, (nH + nKV) * D:].reshape(T, nKV, D)
    assert (q_out.float() - plain(q, qw)).abs().max() <= tol(dtype, 4.0)
    want_k = plain(k, kw)
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for t in range(T):
        p, r = int(positions[t]), int(seq[t])
        pg = int(table[r, p // page])
        assert (_get(kp, pg, p % page).float() - want_k[t]).abs().max() <= tol(dtype, 4.0)
        assert torch.equal(_get(vp, pg, p % page), v[t])
        written[pg, p % page] = True
    unwritten = ~written.to(DEV)[:, None, :].expand(-1, nKV, -1)
    assert float(kp[unwritten].abs().max()) == 0 and float(vp[unwritten].abs().max()) == 0
    # q only (a layer that reads another layer's cache)
    q_only = K().qknorm_rope_kvwrite(qkv[:, :nH * D], nH, nKV, D, qw, kw, eps, cos, sin, rot, positions, None, None,
                                     None, None, False, interleaved=interleaved)
    assert torch.equal(q_only, q_out)
    # a bad page id is reported, not written
    bad = table.clone()
    bad[1, 0] = 99
    K().qknorm_rope_kvwrite(qkv, nH, nKV, D, qw, kw, eps, cos, sin, rot, positions, seq, bad, kp, vp, True, status)
    assert int(status.item()) != 0


@pytest.mark.parametrize("nH,nKV,D,rot", [(32, 8, 128, 128), (6, 2, 64, 64), (9, 3, 128, 64), (7, 1, 64, 32), (8, 4, 128, 0)])
@pytest.mark.parametrize("norm,interleaved", [(True, False), (False, False), (True, True)])
def test_qknorm_rope_kvwrite_many_tokens(nH, nKV, D, rot, norm, interleaved):
    # A prompt step's rows go through the form of the kernel that takes eight heads of a token together (groups
    # that hold queries and keys, keys and values, or run past the last head); the same rows in portions of fewer
    # than 256 tokens, and whole with that form switched off, go through the one-head form, which the test above
    # holds against the formulas: all must agree bit for bit, padding rows of a captured step and a bad page included.
    T, page, eps, theta = 700, 16, 1e-6, 10000.0
    dtype = torch.bfloat16
    qkv = rnd(T, (nH + 2 * nKV) * D + 8, dtype=dtype, seed=5)[:, 8:]            # rows of a wider tensor
    qw, kw = (1 + 0.2 * rnd(D, seed=2), 1 + 0.2 * rnd(D, seed=3)) if norm else (None, None)
    cos = sin = None
    if rot:
        inv = torch.tensor([1.0 / theta ** (i / rot) for i in range(0, rot, 2)], dtype=torch.float64).float()
        ang = torch.arange(512, dtype=torch.float32)[:, None] * inv[None]
        cos, sin = ang.cos().to(DEV), ang.sin().to(DEV)
    # three requests of 300, 250 and 140 tokens and ten padding rows; pages dealt out in a scrambled order
    lens = [300, 250, 140]
    pos = torch.cat([torch.arange(n) for n in lens] + [torch.zeros(10, dtype=torch.long)]).to(torch.int32).to(DEV)
    seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)] + [torch.full((10,), -1)]).to(torch.int32).to(DEV)
    per = -(-max(lens) // page)
    perm = torch.randperm(3 * per + 5, generator=torch.Generator().manual_seed(9)).to(torch.int32)
    table = perm[:3 * per].reshape(3, per).to(DEV)
    num_pages = 3 * per + 5

    def run(rows, table_):
        kp = torch.zeros(num_pages, nKV, page, D, dtype=dtype, device=DEV)
        vp = torch.zeros_like(kp)
        st = torch.zeros(1, dtype=torch.int32, device=DEV)
        outs = []
        for a, b in rows:
            outs.append(K().qknorm_rope_kvwrite(qkv[a:b], nH, nKV, D, qw, kw, eps, cos, sin, rot, pos[a:b], seq[a:b], table_, kp, vp,
                                                True, st, interleaved=interleaved))
        return torch.cat(outs), kp, vp, int(st.item())

    from prelude_b200.ops.library import library
    whole = run([(0, T)], table)
    parts = run([(a, min(a + 200, T)) for a in range(0, T, 200)], table)
    before = library().pb_rope_set_heads_min_tokens(1 << 30)
    try:
        one_head = run([(0, T)], table)
    finally:
        library().pb_rope_set_heads_min_tokens(before)
    assert whole[3] == 0 and parts[3] == 0 and one_head[3] == 0
    assert torch.equal(whole[1], one_head[1]) and torch.equal(whole[2], one_head[2])
    live = (seq >= 0)
    assert torch.equal(whole[0][live], parts[0][live]) and torch.equal(whole[0][live], one_head[0][live])
    assert torch.equal(whole[1], parts[1]) and torch.equal(whole[2], parts[2])
    assert float(whole[1].abs().max()) > 0 and float(whole[2].abs().max()) > 0
    q_only = K().qknorm_rope_kvwrite(qkv[:, :nH * D], nH, nKV, D, qw, kw, eps, cos, sin, rot, pos, None, None, None, None, False,
                                     interleaved=interleaved)
    assert torch.equal(q_only[live], whole[0][live])
    bad = table.clone()
    bad[1, 3] = num_pages + 7                                                    # request 1, positions 48..63
    wb, pb_ = run([(0, T)], bad), run([(a, min(a + 200, T)) for a in range(0, T, 200)], bad)
    assert wb[3] == 2 and pb_[3] == 2
    assert torch.equal(wb[1], pb_[1]) and torch.equal(wb[2], pb_[2]) and torch.equal(wb[0][live], pb_[0][live])


def test_kernels_refuse_what_they_cannot_do():
    from prelude_b200.ops.library import KernelLibraryError
    q = rnd(1, 2, 272)
    kp = torch.zeros(2, 2, 4, 272, device=DEV)
    one = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelLibraryError, match="head_dim"):
        K().paged_attention_ref(q, kp, kp, one, one, torch.zeros(1, 1, dtype=torch.int32, device=DEV), 1.0)
    with pytest.raises(KernelLibraryError, match="rotary_dim"):
        K().qknorm_rope_kvwrite(rnd(1, 64), 2, 1, 16, None, None, 0.0, torch.zeros(4, 9, device=DEV),
                                torch.zeros(4, 9, device=DEV), 18, one, one, torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                torch.zeros(1, 1, 4, 16, device=DEV), torch.zeros(1, 1, 4, 16, device=DEV), True)
    with pytest.raises(KernelLibraryError):
        K().gemm_ref(rnd(2, 3), rnd(4, 5))
    with pytest.raises(KernelLibraryError, match="float32 or bfloat16"):
        K().silu_mul(torch.zeros(2, 4, dtype=torch.float16, device=DEV))


@pytest.mark.parametrize("R,V", [(1, 7), (5, 331), (3, 151936), (64, 1000)])
def test_argmax_ties_go_to_the_smaller_index(R, V):
    logits = rnd(R, V, seed=9)
    logits[0, V // 2] = 50.0
    logits[0, V - 1] = 50.0
    if R > 1:
        logits[1, :] = 0.25                                  # all equal
    got = K().argmax(logits).cpu()
    want = torch.stack([torch.argmax(row) for row in logits.cpu()])
    assert got.tolist() == want.tolist() and got[0] == V // 2 and (R == 1 or got[1] == 0)
    wide = rnd(R, V + 9, seed=10)                            # rows of a wider tensor
    assert K().argmax(wide[:, :V]).tolist() == torch.argmax(wide[:, :V], -1).tolist()


def _philox_host(seed, counter):
    """Philox4x32-10 restated in Python (Salmon et al. 2011)."""
    M0, M1, W0, W1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    c = [counter & mask, (counter >> 32) & mask, 0, 0]
    k0, k1 = seed & mask, (seed >> 32) & mask
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c[3] ^ k1) & mask, p0 & mask]
        k0, k1 = (k0 + W0) & mask, (k1 + W1) & mask
    return (c[0] >> 8) / 16777216.0


def test_philox_matches_its_definition():
    # known answer: counter 0, key 0 -> first word 0x6627e8d5 (Random123 test vectors)
    assert int(_philox_host(0, 0) * 16777216) == 0x6627e8d5 >> 8
    for seed, ctr in [(0, 0), (42, 0), (42, 1), (2**40 + 3, 2**33 + 7), (2**63 - 1, 12345)]:
        assert K().philox_uniform(seed, ctr) == pytest.approx(_philox_host(seed, ctr), abs=0)


@pytest.mark.parametrize("V", [331, 5000, 151936])
def test_sampling_follows_the_distribution_it_is_given(V):
    R = 6
    logits = rnd(R, V, seed=11, scale=2.0)
    temps = torch.tensor([0.0, 0.8, 1.0, 0.3, 1e-9, 2.0], device=DEV)
    seeds = torch.tensor([1, 2, 3, 4, 5, 6], dtype=torch.int64, device=DEV)
    ctrs = torch.tensor([0, 1, 2, 3, 4, 5], dtype=torch.int64, device=DEV)
    got = K().sample(logits, temps, seeds, ctrs).tolist()
    for r in range(R):
        row = logits[r].cpu().double()
        if temps[r] < 1e-7:
            assert got[r] == int(torch.argmax(row))
            continue
        p = torch.exp((row - row.max()) / float(temps[r]))
        cum = torch.cumsum(p, 0)
        u = _philox_host(int(seeds[r]), int(ctrs[r]))
        target = u * float(cum[-1])
        want = int(torch.searchsorted(cum, torch.tensor(target, dtype=torch.float64), right=True))
        # float32 against float64 sums: the pick may fall one boundary away when the draw lands on it
        lo = float(cum[got[r] - 1]) if got[r] > 0 else 0.0
        assert got[r] == want or abs(target - lo) < 1e-4 * float(cum[-1]) or abs(target - float(cum[got[r]])) < 1e-4 * float(cum[-1])
    assert K().sample(logits, temps, seeds, ctrs).tolist() == got          # same seeds, same tokens
    probs = K().softmax_temperature(logits, torch.clamp(temps, min=0.1))
    want = torch.softmax(logits.double() / torch.clamp(temps, min=0.1).double()[:, None], -1)
    assert (probs.double() - want).abs().max() < 1e-6 and torch.allclose(probs.sum(-1), torch.ones(R, device=DEV), atol=1e-5)


def test_sampling_frequencies():
    V, n = 17, 4000
    logits = rnd(1, V, seed=12).repeat(n, 1).contiguous()
    temps = torch.full((n,), 0.7, device=DEV)
    seeds = torch.full((n,), 99, dtype=torch.int64, device=DEV)
    ctrs = torch.arange(n, dtype=torch.int64, device=DEV)
    got = K().sample(logits, temps, seeds, ctrs)
    freq = torch.bincount(got.long(), minlength=V).float() / n
    want = torch.softmax(logits[0] / 0.7, -1)
    assert (freq - want).abs().max() < 0.03


# ---------------------------------------------------------------------------------------
# tensor-core attention (bfloat16): prompt portions and decode steps, through the dispatch
# ---------------------------------------------------------------------------------------
def _batch_for(requests, page, num_pages, nKV, D, seed, trimmed_below=None):
    """requests: list of (context_len, q_len): the last q_len tokens are this step's queries.
    Returns (batch, k, v lists, pages, kp, vp)."""
    from prelude_b200.engine.batch import StepItem, build_step_batch
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    kp = torch.full((num_pages, nKV, page, D), float("nan"), dtype=torch.bfloat16, device=DEV)
    vp = torch.full_like(kp, float("nan"))
    ks, vs, tables, items = [], [], [], []
    for i, (ctx, qn) in enumerate(requests):
        k, v = rnd(ctx, nKV, D, dtype=torch.bfloat16, seed=seed + 10 * i + 1), rnd(ctx, nKV, D, dtype=torch.bfloat16, seed=seed + 10 * i + 2)
        n = -(-ctx // page)
        pages, perm = perm[:n], perm[n:]
        for j in range(ctx):
            _put(kp, pages[j // page], j % page, k[j])
            _put(vp, pages[j // page], j % page, v[j])
        if trimmed_below is not None:                       # pages wholly below this position have been given back
            pages = [-1 if (pi + 1) * page <= trimmed_below[i] else pg for pi, pg in enumerate(pages)]
        ks.append(k); vs.append(v); tables.append(pages)
        items.append(StepItem(i, [0] * qn, ctx - qn))
    batch = build_step_batch(items, {0: tables}, list(range(len(requests))), torch.device(DEV), 10, 1 << 20)
    return batch, ks, vs, kp, vp


def _check_dispatch(requests, nH, nKV, D, page, window, seed=0, trimmed_below=None, tolerance=None):
    from prelude_b200.ops.attention import paged_attention
    batch, ks, vs, kp, vp = _batch_for(requests, page, max(600, sum(-(-c // page) for c, _ in requests) + 8), nKV, D, seed, trimmed_below)
    q = rnd(batch.n_tokens, nH, D, dtype=torch.bfloat16, seed=seed + 99)
    got = paged_attention(q, kp, vp, batch, 0, 1 / math.sqrt(D), window)
    assert int(batch.status.item()) == 0
    row = 0
    for i, (ctx, qn) in enumerate(requests):
        want = _attention_plain(q[row:row + qn], ks[i], vs[i], list(range(ctx - qn, ctx)), 1 / math.sqrt(D), window)
        diff = (got[row:row + qn].double() - want).abs().max()
        assert diff <= (tolerance or tol(torch.bfloat16, 4.0)), (i, ctx, qn, float(diff))
        row += qn
    assert not torch.isnan(got.float()).any()
    return got


@pytest.mark.parametrize("nH,nKV,D,page", [(4, 2, 16, 4), (6, 2, 32, 8), (5, 1, 48, 16), (8, 8, 64, 16), (3, 3, 80, 16),
                                           (32, 8, 128, 16), (2, 1, 256, 32), (16, 2, 128, 16), (7, 7, 112, 16),
                                           (4, 2, 64, 24), (8, 2, 128, 48), (4, 1, 128, 64), (6, 3, 64, 128),
                                           (4, 4, 192, 16), (4, 1, 128, 8), (2, 2, 256, 40)])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("kernel", ["auto", "mma"])
def test_attention_prefill_tensor_cores(monkeypatch, nH, nKV, D, page, window, kernel):
    # whole prompts, a portion that continues a cached prefix, single tokens in between, a two-token portion;
    # "auto" takes the tcgen05 kernel where it takes the shape, "mma" keeps every shape on the mma.sync kernel
    from prelude_b200.ops import attention
    monkeypatch.setattr(attention, "PREFILL_KERNEL", kernel)
    requests = [(83, 83), (200, 37), (150, 1), (2, 2), (130, 129), (65, 1), (64, 64)]
    _check_dispatch(requests, nH, nKV, D, page, window)


@pytest.mark.parametrize("nH,nKV,D,page", [(3, 3, 64, 8), (4, 2, 128, 16), (8, 2, 64, 32), (16, 2, 128, 64), (16, 1, 64, 128),
                                           (32, 1, 128, 256), (2, 2, 128, 64), (32, 8, 128, 16)])
@pytest.mark.parametrize("window", [None, 100, 300])
def test_attention_prefill_tcgen05(monkeypatch, nH, nKV, D, page, window):
    """The tcgen05 kernel alone, at every group size it takes (1 to 32 query heads per key/value head), both head
    sizes and pages from 8 to 256 tokens: portions longer and shorter than a block's tokens, a long cached prefix,
    portions that end one key before, at and after a tile's edge, and single tokens."""
    from prelude_b200.ops import attention
    from prelude_b200.ops import library as L
    assert L.library().pb_attention_prefill_tc_supported(nH, nKV, D, page, 1)
    monkeypatch.setattr(attention, "PREFILL_KERNEL", "tc")
    requests = [(300, 300), (700, 90), (127, 127), (128, 128), (129, 129), (513, 1), (1000, 260), (5, 5), (257, 2)]
    got_tc = _check_dispatch(requests, nH, nKV, D, page, window, seed=3)
    monkeypatch.setattr(attention, "PREFILL_KERNEL", "mma")
    got_mma = _check_dispatch(requests, nH, nKV, D, page, window, seed=3)
    assert (got_tc.float() - got_mma.float()).abs().max() <= tol(torch.bfloat16, 4.0)


@pytest.mark.parametrize("nH,nKV,D,page", [(32, 8, 128, 16), (4, 4, 64, 8), (16, 1, 128, 64)])
@pytest.mark.parametrize("requests", [[(5, 5)], [(33, 33)], [(300, 3)], [(64, 64), (2, 2)]], ids=str)
def test_attention_prefill_tcgen05_on_steps_with_few_tokens(monkeypatch, nH, nKV, D, page, requests):
    # the query box of the tensor map is then taller than the query tensor
    from prelude_b200.ops import attention
    monkeypatch.setattr(attention, "PREFILL_KERNEL", "tc")
    _check_dispatch(requests, nH, nKV, D, page, None)


def test_attention_prefill_tcgen05_refuses_what_it_does_not_take():
    from prelude_b200.ops import library as L
    lib = L.library()
    assert not lib.pb_attention_prefill_tc_supported(6, 2, 128, 16, 1)       # three query heads per key/value head
    assert not lib.pb_attention_prefill_tc_supported(8, 2, 96, 16, 1)        # head size
    assert not lib.pb_attention_prefill_tc_supported(8, 2, 128, 24, 1)       # pages that do not tile 128 keys
    assert not lib.pb_attention_prefill_tc_supported(8, 2, 128, 16, 0)       # pages that are not permuted
    assert lib.pb_attention_prefill_tc_tile_tokens(32, 8) == 64
    t = torch.zeros(64, dtype=torch.bfloat16, device=DEV)
    i = torch.zeros(8, dtype=torch.int32, device=DEV)
    code = lib.pb_attention_prefill_tc_bf16(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), i.data_ptr(), 1, i.data_ptr(),
                                            i.data_ptr(), i.data_ptr(), i.data_ptr(), i.data_ptr(), i.data_ptr(), 1, 24, 1, 1, 8, 2,
                                            128, 0.1, 0, 1, i.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code != 0 and "not taken" in L.last_error()


@pytest.mark.parametrize("nH,nKV,D,page", [(4, 2, 16, 4), (6, 2, 32, 8), (5, 1, 48, 16), (8, 8, 64, 16), (3, 3, 80, 16),
                                           (32, 8, 128, 16), (2, 1, 256, 32), (16, 1, 128, 16), (7, 7, 112, 16),
                                           (4, 2, 64, 24), (8, 2, 128, 48), (4, 1, 128, 64), (6, 3, 64, 128),
                                           (4, 4, 192, 16), (4, 1, 128, 8), (2, 2, 256, 40)])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("splits,cluster", [(None, True), (1, True), (3, True), (8, True), (16, True), (None, False), (3, False), (20, True)],
                         ids=["plan", "1", "3", "8", "16", "plan-scratch", "3-scratch", "20-scratch"])
def test_attention_decode_tensor_cores(monkeypatch, nH, nKV, D, page, window, splits, cluster):
    # the parts of a (token, head)'s splits are added up through the shared memory of a thread-block cluster (up to
    # 16 splits, where the device places such a cluster) or through scratch memory (more splits, or clusters off)
    from prelude_b200.ops import attention
    from prelude_b200.ops import library as L
    if splits is not None:
        monkeypatch.setattr(attention, "decode_splits", lambda *a, **k: splits)
    requests = [(1, 1), (2, 1), (63, 1), (64, 1), (65, 1), (128, 1), (129, 1), (500, 1), (777, 1)]
    L.library().pb_attention_decode_set_cluster(1 if cluster else 0)
    try:
        for _ in range(2):                                  # twice: the scratch way leaves its counters at zero
            _check_dispatch(requests, nH, nKV, D, page, window)
    finally:
        L.library().pb_attention_decode_set_cluster(1)


def test_attention_with_pages_that_a_window_has_given_back():
    window = 40
    reqs = [(300, 1), (170, 1)]
    _check_dispatch(reqs, 8, 2, 64, 16, window, trimmed_below=[300 - window, 170 - window])
    reqs = [(300, 30), (170, 2)]                       # portions: the first query still reads from ctx - q - window + 1
    _check_dispatch(reqs, 8, 2, 64, 16, window, trimmed_below=[300 - 30 - window + 1, 170 - 2 - window + 1])


@pytest.mark.parametrize("decode", [True, False])
@pytest.mark.parametrize("where", ["far", "page_edge", "tile_edge", "window_first", "just_outside_window", "self"])
def test_tensor_core_attention_finds_the_one_key_that_matters(monkeypatch, decode, where):
    from prelude_b200.ops import attention
    from prelude_b200.ops.attention import paged_attention
    monkeypatch.setattr(attention, "decode_splits", lambda *a, **k: 5)
    nH, nKV, D, page, L, window = 8, 2, 128, 16, 700, 200
    qn = 1 if decode else 3
    batch, ks, vs, kp, vp = _batch_for([(L, qn)], page, 64, nKV, D, seed=4)
    pos = L - 1
    target = {"far": 2, "page_edge": 15 * page, "tile_edge": 64 * 7 - 1, "window_first": pos - window + 1,
              "just_outside_window": pos - window, "self": pos}[where]
    unit = torch.zeros(D, device=DEV)
    unit[9] = 1.0
    q = rnd(qn, nH, D, dtype=torch.bfloat16, seed=5, scale=0.05)
    q[-1] = (unit * 30).to(torch.bfloat16)
    pg = int(batch.block_tables[0][0, target // page])
    kp[:, :, :, :] = (kp.float() * 0.05).to(torch.bfloat16)
    _put(kp, pg, target % page, (unit * 30).to(torch.bfloat16).expand(nKV, D))      # score 900 / sqrt(128) = 80 against ~0
    use_window = window if where in ("window_first", "just_outside_window") else None
    got = paged_attention(q, kp, vp, batch, 0, 1 / math.sqrt(D), use_window)
    hit = (got[-1, 0].float() - vs[0][target, 0].float()).abs().max() < 0.06
    assert bool(hit) == (where != "just_outside_window")
    ref = K().paged_attention_ref(q, kp, vp, batch.positions, batch.token_seq, batch.block_tables[0], 1 / math.sqrt(D), use_window)
    assert (got.float() - ref.float()).abs().max() <= tol(torch.bfloat16, 4.0)


@pytest.mark.parametrize("qn", [1, 130], ids=["decode", "portion"])
@pytest.mark.parametrize("target", [2, 16384, 33000 - 131])
def test_tensor_core_attention_finds_the_one_key_that_matters_in_a_long_context(qn, target):
    # 33,000 keys, 2,063 pages in a scrambled order: the planner's own splits and clusters for the decode kernel, a
    # block table far longer than the window of it that the prompt kernel keeps in registers; one key (an early
    # one, one at 16,384, the last that the portion's first query may see)
    # carries all the weight of the last query's heads
    from prelude_b200.ops.attention import paged_attention
    nH, nKV, D, page, L = 8, 2, 128, 16, 33000
    batch, ks, vs, kp, vp = _batch_for([(L, qn)], page, L // page + 8, nKV, D, seed=6)
    unit = torch.zeros(D, device=DEV)
    unit[9] = 1.0
    q = rnd(qn, nH, D, dtype=torch.bfloat16, seed=5, scale=0.05)
    q[-1] = (unit * 30).to(torch.bfloat16)
    q[0] = (unit * 30).to(torch.bfloat16)
    kp[:, :, :, :] = (kp.float() * 0.05).to(torch.bfloat16)
    pg = int(batch.block_tables[0][0, target // page])
    _put(kp, pg, target % page, (unit * 30).to(torch.bfloat16).expand(nKV, D))      # score 900 / sqrt(128) = 80 against ~0
    got = paged_attention(q, kp, vp, batch, 0, 1 / math.sqrt(D), None)
    assert (got[-1, 0].float() - vs[0][target, 0].float()).abs().max() < 0.06
    if target <= L - qn:                                   # the portion's first query sees it too
        assert (got[0, 3].float() - vs[0][target, 0].float()).abs().max() < 0.06
    ref = K().paged_attention_ref(q, kp, vp, batch.positions, batch.token_seq, batch.block_tables[0], 1 / math.sqrt(D), None)
    assert (got.float() - ref.float()).abs().max() <= tol(torch.bfloat16, 4.0)


def test_tensor_core_attention_refuses_or_falls_back():
    from prelude_b200.ops.attention import tensor_core_shape_ok
    assert tensor_core_shape_ok(32, 8, 128, True) and tensor_core_shape_ok(64, 1, 128, False)
    assert not tensor_core_shape_ok(64, 1, 128, True) and not tensor_core_shape_ok(8, 8, 24, False)
    _check_dispatch([(90, 1), (33, 1)], 40, 2, 64, 16, None)      # 20 heads per group: the plain kernel serves the decode step
    _check_dispatch([(90, 5)], 8, 8, 24, 16, None)                # head size 24: plain kernel


# ---------------------------------------------------------------------------------------
# the weight-streaming product for decode steps
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("N,K_", [(2560, 4096), (19456, 2560), (6144, 2560), (2560, 9728), (48, 64), (16, 32),
                                  (176, 96), (1008, 1504), (7, 32), (151936, 2560), (333, 2064), (333, 2080)])
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
def test_gemm_stream(M, N, K_):
    from prelude_b200.ops.linear import gemm_stream, stream_takes, tc_status
    x, w, b = rnd(M, K_, dtype=torch.bfloat16, seed=21), rnd(N, K_, dtype=torch.bfloat16, seed=22, scale=0.05), rnd(N, seed=23)
    if not stream_takes(x, w):              # K no multiple of 32, or x too long to fit beside the ring
        assert K_ % 32 or (M > 8 and K_ > 6000)
        return
    want = x.double() @ w.double().T
    scale = float(want.abs().max())
    got = gemm_stream(x, w)
    assert (got.double() - want).abs().max() <= tol(torch.bfloat16, scale)
    assert torch.equal(gemm_stream(x, w), got)
    got32 = gemm_stream(x, w, b, torch.float32)
    assert got32.dtype == torch.float32
    assert (got32.double() - (want + b.double())).abs().max() <= 2e-3 * max(1.0, scale)
    if M > 1:            # a row does not depend on the rest of the batch, beyond rounding (K is cut differently)
        alone = gemm_stream(x[M - 1:M].contiguous(), w)
        assert (alone.double() - got[M - 1:M].double()).abs().max() <= tol(torch.bfloat16, scale)
    wide = rnd(M, K_ + 64, dtype=torch.bfloat16, seed=24)            # x as a view into a wider tensor
    assert torch.equal(gemm_stream(wide[:, 32:32 + K_], w), gemm_stream(wide[:, 32:32 + K_].contiguous(), w))
    assert int(tc_status(x.device).item()) == 0


@pytest.mark.parametrize("M,I,K_", [(8, 9728, 2560), (1, 200, 64), (16, 77, 96), (3, 8, 32), (5, 1000, 1504)])
def test_gemm_stream_gated(M, I, K_):
    # silu(x Wg^T) * (x Wu^T) from the merged weight, against the two-step computation in float64
    from prelude_b200.ops.linear import gated_linear_silu, gemm_stream
    x, w = rnd(M, K_, dtype=torch.bfloat16, seed=31), rnd(2 * I, K_, dtype=torch.bfloat16, seed=32, scale=0.05)
    g, u = x.double() @ w[:I].double().T, x.double() @ w[I:].double().T
    want = g / (1 + torch.exp(-g)) * u
    got = gemm_stream(x, w, gated=True)
    assert got.shape == (M, I) and got.dtype == torch.bfloat16
    assert (got.double() - want).abs().max() <= tol(torch.bfloat16, float(want.abs().max()))
    assert torch.equal(gated_linear_silu(x, w), got)
    assert gated_linear_silu(rnd(40, K_, dtype=torch.bfloat16), w) is None      # too many rows: the caller takes two steps


# ---------------------------------------------------------------------------------------
# the paired-block tcgen05 product for prompt steps
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K_", [(2048, 2560, 4096), (1024, 6144, 2560), (256, 256, 64), (300, 520, 328), (77, 1000, 72),
                                    (515, 264, 2056), (1, 8, 8), (1000, 40003, 96)])
@pytest.mark.parametrize("max_pairs", [0, 3])
def test_gemm_pair(M, N, K_, max_pairs):
    # tiles that end inside the matrix in every direction, one pair that walks many tiles, more pairs than tiles
    from prelude_b200.ops.linear import gemm_pair, pair_takes, tc_status
    x, w, b = rnd(M, K_, dtype=torch.bfloat16, seed=41), rnd(N, K_, dtype=torch.bfloat16, seed=42, scale=0.05), rnd(N, seed=43)
    assert pair_takes(x, w)
    want = x.double() @ w.double().T
    scale = float(want.abs().max())
    got = gemm_pair(x, w, max_pairs=max_pairs)
    assert got.shape == (M, N) and got.dtype == torch.bfloat16
    assert (got.double() - want).abs().max() <= tol(torch.bfloat16, scale)
    assert torch.equal(gemm_pair(x, w, max_pairs=max_pairs), got)
    assert torch.equal(gemm_pair(x, w, max_pairs=5), got)                 # who computes a tile does not change it
    with_bias = gemm_pair(x, w, b, max_pairs=max_pairs)
    assert (with_bias.double() - (want + b.double())).abs().max() <= tol(torch.bfloat16, scale + float(b.abs().max()))
    if M > 1:           # a row does not depend on the rows beside it
        assert torch.equal(gemm_pair(x[M - 1:M].contiguous(), w), got[M - 1:M])
    wide = rnd(M, K_ + 64, dtype=torch.bfloat16, seed=44)                  # x and the result as views into wider tensors
    out = torch.full((M, N + 24), 7.0, dtype=torch.bfloat16, device="cuda")
    gemm_pair(wide[:, 32:32 + K_], w, out=out[:, 8:8 + N])
    assert torch.equal(out[:, 8:8 + N], gemm_pair(wide[:, 32:32 + K_].contiguous(), w))
    assert bool((out[:, :8] == 7).all()) and bool((out[:, 8 + N:] == 7).all())
    assert int(tc_status(x.device).item()) == 0


@pytest.mark.parametrize("M,I,K_", [(2048, 9728, 2560), (768, 1000, 264), (256, 128, 64), (300, 77, 96), (5, 8, 32), (1030, 200, 1504)])
def test_gemm_pair_gated(M, I, K_):
    # silu(x Wg^T) * (x Wu^T) from the merged weight, against the two-step computation in float64
    from prelude_b200.ops.linear import PAIR_MIN_ROWS, gated_linear_silu, gemm_pair, tc_status
    x, w = rnd(M, K_, dtype=torch.bfloat16, seed=51), rnd(2 * I, K_, dtype=torch.bfloat16, seed=52, scale=0.05)
    g, u = x.double() @ w[:I].double().T, x.double() @ w[I:].double().T
    want = g / (1 + torch.exp(-g)) * u
    got = gemm_pair(x, w, gated=True)
    assert got.shape == (M, I) and got.dtype == torch.bfloat16
    assert (got.double() - want).abs().max() <= tol(torch.bfloat16, float(want.abs().max()))
    assert torch.equal(gemm_pair(x, w, gated=True, max_pairs=2), got)
    if M >= PAIR_MIN_ROWS:
        assert torch.equal(gated_linear_silu(x, w), got)                  # a prompt step's projection goes this way
    assert int(tc_status(x.device).item()) == 0


@pytest.mark.parametrize("nH,nKV,D", [(32, 8, 128), (5, 1, 64), (6, 2, 64), (3, 1, 256), (9, 3, 128)])
@pytest.mark.parametrize("norm", [True, False])
def test_gemm_pair_with_heads_epilogue(nH, nKV, D, norm):
    # The merged q/k/v projection with norm, rotation and cache write in the product's epilogue against the product
    # followed by the kernel that the tests above hold against the formulas: the same queries and the same pages
    # within the rounding of the projection to bfloat16 that the one-kernel form leaves out; tiles that end inside
    # the heads' columns, padding rows of a captured step, a token without a page, a position outside the tables.
    from prelude_b200.ops.linear import qkv_heads
    T, H, page, eps, theta = 600, 328, 16, 1e-6, 10000.0
    x = rnd(T, H, dtype=torch.bfloat16, seed=61)
    w = rnd((nH + 2 * nKV) * D, H, dtype=torch.bfloat16, seed=62, scale=0.06)
    qw, kw = (1 + 0.2 * rnd(D, seed=2), 1 + 0.2 * rnd(D, seed=3)) if norm else (None, None)
    inv = torch.tensor([1.0 / theta ** (i / D) for i in range(0, D, 2)], dtype=torch.float64).float()
    ang = torch.arange(400, dtype=torch.float32)[:, None] * inv[None]
    cos, sin = ang.cos().to(DEV), ang.sin().to(DEV)
    lens = [290, 200, 100]
    pos = torch.cat([torch.arange(n) for n in lens] + [torch.zeros(10, dtype=torch.long)]).to(torch.int32).to(DEV)
    seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)] + [torch.full((10,), -1)]).to(torch.int32).to(DEV)
    per = -(-max(lens) // page)
    num_pages = 3 * per + 5
    table = torch.randperm(num_pages, generator=torch.Generator().manual_seed(9)).to(torch.int32)[:3 * per].reshape(3, per).to(DEV)
    live = seq >= 0

    def run(fused, table_, pos_, write_kv=True):
        kp = torch.zeros(num_pages, nKV, page, D, dtype=torch.bfloat16, device=DEV)
        vp = torch.zeros_like(kp)
        st = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = torch.zeros(T, nH, D, dtype=torch.bfloat16, device=DEV)
        qkv_heads(x, w, None, nH, nKV, D, qw, kw, eps, cos, sin, D, False, pos_, seq if write_kv else None, table_ if write_kv else None,
                  kp if write_kv else None, vp if write_kv else None, write_kv, st, out, force=fused)
        return out, kp, vp, int(st.item())

    one, two = run(True, table, pos), run(False, table, pos)
    assert one[3] == 0 and two[3] == 0
    scale = float(two[0].float().abs().max())
    for a, b in ((one[0][live], two[0][live]), (one[1], two[1]), (one[2], two[2])):
        assert (a.float() - b.float()).abs().max() <= tol(torch.bfloat16, scale)
    assert float(one[1].abs().max()) > 0 and float(one[2].abs().max()) > 0
    assert torch.equal(one[1] == 0, two[1] == 0) or float(((one[1] == 0) != (two[1] == 0)).float().mean()) < 1e-3   # the same places written
    assert torch.equal(one[0][~live], torch.zeros_like(one[0][~live]))                 # padding rows store nothing
    assert torch.equal(run(True, table, pos)[0], one[0])
    q_only = run(True, table, pos, write_kv=False)
    assert q_only[3] == 0 and torch.equal(q_only[0][live], one[0][live])
    bad = table.clone()
    bad[1, 3] = num_pages + 7
    b1, b2 = run(True, bad, pos), run(False, bad, pos)
    assert b1[3] == 2 and b2[3] == 2
    assert torch.equal(b1[1] == 0, b2[1] == 0) or float(((b1[1] == 0) != (b2[1] == 0)).float().mean()) < 1e-3
    far = pos.clone()
    far[5] = 400                                                                       # outside the tables
    assert run(True, table, far)[3] != 0 and run(False, table, far)[3] != 0


def test_gemm_pair_finds_the_one_weight_that_matters():
    # one large product at chosen places of M, N and K, everything else small: a lost stage, row or column shows
    from prelude_b200.ops.linear import gemm_pair
    M, N, K_ = 700, 1300, 1096
    x, w = rnd(M, K_, dtype=torch.bfloat16, seed=1, scale=0.01), rnd(N, K_, dtype=torch.bfloat16, seed=2, scale=0.01)
    for (m, n, k) in [(0, 0, 0), (M - 1, N - 1, K_ - 1), (127, 127, 63), (128, 128, 64), (255, 255, 383), (256, 256, 384),
                      (511, 1279, 1087), (640, 1280, 1088), (129, 383, 447), (383, 129, 448)]:
        x2, w2 = x.clone(), w.clone()
        x2[m, k], w2[n, k] = 8.0, 8.0
        got = gemm_pair(x2, w2, max_pairs=4)
        assert abs(float(got[m, n]) - 64.0) < 1.0
        got[m, n] = 0
        assert float(got.abs().max()) < 1.0


def test_gemm_pair_refuses_other_shapes_and_linear_goes_on():
    from prelude_b200.ops.library import KernelLibraryError
    from prelude_b200.ops.linear import gemm_pair, linear, pair_takes
    x, w = rnd(300, 68, dtype=torch.bfloat16), rnd(40, 68, dtype=torch.bfloat16)      # rows of 136 bytes: no tensor map
    assert not pair_takes(x, w)
    with pytest.raises(KernelLibraryError, match="not taken"):
        gemm_pair(x, w)
    want = x.double() @ w.double().T
    assert (linear(x, w).double() - want).abs().max() <= tol(torch.bfloat16, float(want.abs().max()))
    assert not pair_takes(rnd(300, 64, dtype=torch.bfloat16), rnd(41, 64, dtype=torch.bfloat16), gated=True)   # gate rows != up rows
    with pytest.raises(KernelLibraryError, match="no bias"):
        gemm_pair(rnd(300, 64, dtype=torch.bfloat16), rnd(40, 64, dtype=torch.bfloat16), rnd(20), gated=True)


def test_gemm_stream_finds_the_one_weight_that_matters():
    # one large product at the far end of K and of N, everything else small: a lost chunk or row shows
    from prelude_b200.ops.linear import gemm_stream
    M, N, K_ = 5, 2563 - 3, 4096
    x, w = rnd(M, K_, dtype=torch.bfloat16, seed=1, scale=0.01), rnd(N, K_, dtype=torch.bfloat16, seed=2, scale=0.01)
    for (m, n, k) in [(0, 0, 0), (4, N - 1, K_ - 1), (2, 1297, 2047), (3, 17, 2048), (1, N - 17, 2815), (0, 8, 31), (4, 7, 32)]:
        x2, w2 = x.clone(), w.clone()
        x2[m, k], w2[n, k] = 8.0, 8.0
        got = gemm_stream(x2, w2)
        assert abs(float(got[m, n]) - 64.0) < 1.0
        got[m, n] = 0
        assert float(got.abs().max()) < 1.0


def test_gemm_stream_refuses_other_shapes_and_linear_falls_back():
    from prelude_b200.ops.library import KernelLibraryError
    from prelude_b200.ops.linear import gemm_stream, linear, stream_takes
    x, w = rnd(4, 72, dtype=torch.bfloat16), rnd(40, 72, dtype=torch.bfloat16)      # K is no multiple of 16
    assert not stream_takes(x, w)
    with pytest.raises(KernelLibraryError, match="not taken"):
        gemm_stream(x, w)
    want = x.double() @ w.double().T
    assert (linear(x, w).double() - want).abs().max() <= tol(torch.bfloat16, float(want.abs().max()))
    assert not stream_takes(rnd(17, 64, dtype=torch.bfloat16), rnd(64, 64, dtype=torch.bfloat16))
    assert stream_takes(rnd(8, 64, dtype=torch.bfloat16), rnd(64, 64, dtype=torch.bfloat16))


