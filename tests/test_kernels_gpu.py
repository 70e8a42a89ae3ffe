"""Each CUDA kernel alone against a plain float32 PyTorch statement of the same
operation, at sizes other than the engine's tiny models use: widths and
vocabularies that are no power of two, head sizes in steps of 16, one kv head
under many query heads, page sizes 8 to 64.  Where random inputs would hide a
fault the inputs are made so that it shows: one far key among hundreds that must
dominate, keys just inside and just outside a window, a value that marks each
page."""

import math

import numpy as np
import pytest
import torch

from paged_llm_rs_b200.errors import KernelError
from paged_llm_rs_b200.kernels import attention_plan, ops
from paged_llm_rs_b200.parts.base import AttentionWork

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(72, 1000), (1024, 50), (33, 7)])
def test_embed(dtype, hidden, vocab):
    g = torch.Generator(device=DEV).manual_seed(0)
    table = torch.randn(vocab, hidden, device=DEV, generator=g).to(dtype)
    tokens = torch.randint(0, vocab, (37,), device=DEV, generator=g, dtype=torch.int32)
    out = torch.empty(37, hidden, device=DEV, dtype=dtype)
    st = status()
    ops.embed(tokens, table, out, st)
    assert torch.equal(out, table[tokens.long()]) and st.item() == 0
    tokens[3] = vocab  # out of range: zeros and a raised status bit, no fault
    ops.embed(tokens, table, out, st)
    assert st.item() == 1 and out[3].abs().sum() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [19, 1100])     # few rows: a CTA a row; many: teams of one to eight warps a row
@pytest.mark.parametrize("width,eps", [(96, 1e-5), (1000, 1e-6), (1024, 1e-6), (2056, 1e-5), (4096, 1e-6), (5120, 1e-6),
                                       (9000, 1e-6), (50, 1e-3)])
def test_rmsnorm_plain_fused_and_gathered(dtype, n, width, eps):
    g = torch.Generator(device=DEV).manual_seed(1)
    x = (torch.randn(n, width, device=DEV, generator=g) * 3).to(dtype)
    d = torch.randn(n, width, device=DEV, generator=g).to(dtype)
    gain = 1 + 0.1 * torch.randn(width, device=DEV, generator=g)

    def ref(v):
        v = v.float()
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * gain

    out = torch.empty_like(x)
    ops.rmsnorm(x, gain, eps, out)
    torch.testing.assert_close(out.float(), ref(x), **tol(dtype))
    # fused residual add: the sum is stored in the stream's dtype and normed from there
    res = x.clone()
    ops.rmsnorm(res, gain, eps, out, delta=d, residual_out=res)
    summed = (x.float() + d.float()).to(dtype)
    assert torch.equal(res, summed)
    torch.testing.assert_close(out.float(), ref(summed), **tol(dtype))
    # gathered rows with a pending add, nothing stored
    rows = torch.randperm(n, device=DEV, generator=g)[:max(3, n // 2)].to(torch.int32)
    res2 = x.clone()
    out3 = torch.full((rows.numel() + 1, width), 7.0, device=DEV, dtype=dtype)
    ops.rmsnorm(res2, gain, eps, out3[:-1], delta=d, rows=rows)
    assert torch.equal(res2, x) and (out3[-1] == 7).all()
    torch.testing.assert_close(out3[:-1].float(), ref(summed[rows.long()]), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [160, 3072, 77])
def test_swiglu(dtype, inter):
    g = torch.Generator(device=DEV).manual_seed(2)
    gu = (torch.randn(11, 2 * inter, device=DEV, generator=g) * 2).to(dtype)
    out = torch.empty(11, inter, device=DEV, dtype=dtype)
    ops.swiglu(gu, out)
    a, b = gu.float()[:, :inter], gu.float()[:, inter:]
    torch.testing.assert_close(out.float(), a * torch.sigmoid(a) * b, **tol(dtype))   # the gate carries the activation


def rope_ref(x, pos, theta, rotary_dim):
    half = rotary_dim // 2
    inv = 1.0 / theta ** (torch.arange(half, dtype=torch.float64) * 2 / rotary_dim)
    ang = pos.double()[:, None] * inv[None]
    c, s = ang.cos().float().to(x.device)[:, None], ang.sin().float().to(x.device)[:, None]
    x1, x2 = x[..., :half], x[..., half:rotary_dim]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, x[..., rotary_dim:]], -1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rot,page", [(6, 3, 48, 48, 8), (8, 1, 32, 16, 16), (16, 8, 128, 128, 64), (4, 4, 80, 80, 16),
                                                (4, 2, 64, 64, 16), (3, 1, 256, 256, 8), (5, 5, 32, 32, 16)])
@pytest.mark.parametrize("T", [21, 301, 1601])     # a lane a chunk of a head (two kernels); very many: a warp a token
def test_qk_norm_rope_kv_write(dtype, nh, nkv, hd, rot, page, T):
    from paged_llm_rs_b200.parts.base import Runtime
    from paged_llm_rs_b200.parts.position import RotaryEncoding
    from paged_llm_rs_b200.parts.spec import PartSpec

    g = torch.Generator(device=DEV).manual_seed(3)
    pages, eps, theta = -(-T // page) + 7, 1e-5, 1e6
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV, generator=g).to(dtype)
    qg = 1 + 0.1 * torch.randn(hd, device=DEV, generator=g)
    kg = 1 + 0.1 * torch.randn(hd, device=DEV, generator=g)
    pos = torch.randint(0, 300, (T,), device=DEV, generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * page, device=DEV, generator=g)[:T].to(torch.int32)
    slots[5] = -1  # a token that is not to be written
    enc = RotaryEncoding(PartSpec("rope", dict(head_dim=hd, rotary_dim=rot, theta=theta, max_positions=300)),
                         Runtime(torch.device(DEV), dtype))
    cos, sin, rdim = enc.rotary()
    kp = torch.zeros(pages, nkv, page, hd, device=DEV, dtype=dtype)
    vp = torch.zeros_like(kp)
    q = torch.empty(T, nh * hd, device=DEV, dtype=dtype)
    st = status()
    ops.qk_norm_rope_kv(qkv, q, qg, kg, eps, cos, sin, rdim, pos, slots, kp, vp, nh, nkv, hd, st)
    assert st.item() == 0

    x = qkv.float().view(T, nh + 2 * nkv, hd)
    norm = lambda v, gain: v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * gain
    q_ref = rope_ref(norm(x[:, :nh], qg), pos.cpu(), theta, rot)       # norm per head, then the rotation
    k_ref = rope_ref(norm(x[:, nh:nh + nkv], kg), pos.cpu(), theta, rot)
    v_ref = x[:, nh + nkv:]                                            # values raw
    torch.testing.assert_close(q.float().view(T, nh, hd), q_ref, **tol(dtype))
    for t in range(T):
        s = slots[t].item()
        if s < 0:
            continue
        torch.testing.assert_close(kp[s // page, :, s % page].float(), k_ref[t], **tol(dtype))
        torch.testing.assert_close(vp[s // page, :, s % page].float(), v_ref[t], **tol(dtype))
    written = torch.zeros(pages * page, dtype=torch.bool)
    written[slots[slots >= 0].long().cpu()] = True
    flat = kp.float().permute(0, 2, 1, 3).reshape(pages * page, -1).abs().sum(-1).cpu()
    assert (flat[~written] == 0).all()          # nothing else was touched


# --- attention -------------------------------------------------------------------------

def attention_ref(q, k, v, scale, window):
    """q [nq, nh, hd] at positions pos0.., k/v [ctx, nkv, hd]; float64."""
    nq, nh, hd = q.shape
    ctx, nkv, _ = k.shape
    pos0 = ctx - nq
    g = nh // nkv
    out = torch.zeros(nq, nh, hd, dtype=torch.float64)
    for h in range(nh):
        s = q[:, h].double() @ k[:, h // g].double().T * scale
        i = torch.arange(nq)[:, None] + pos0
        j = torch.arange(ctx)[None]
        hidden = j > i
        if window:
            hidden |= j <= i - window
        s = s.masked_fill(hidden, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, h // g].double()
    return out


def run_attention(dtype, reqs, nh, nkv, hd, page, window, target_ctas, seed=0, craft=None, kinds=3,
                  raw=False, idle_items=0, min_split_keys=128, multi_min_split_keys=128):
    """reqs: list of (context before the step, query tokens).  Builds a paged cache
    with shuffled pages, runs the kernel, returns (got, want) per request."""
    g = torch.Generator().manual_seed(seed)
    scale = hd ** -0.5
    n_pages = sum(-(-(c + n) // page) for c, n in reqs) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    kp = torch.zeros(n_pages, nkv, page, hd, dtype=dtype)
    vp = torch.zeros_like(kp)
    width = max(-(-(c + n) // page) for c, n in reqs)
    tables = torch.full((len(reqs), width), -1, dtype=torch.int32)
    qs, ks, vs, segs = [], [], [], []
    t0 = 0
    for r, (c, n) in enumerate(reqs):
        total = c + n
        k = torch.randn(total, nkv, hd, generator=g)
        v = torch.randn(total, nkv, hd, generator=g)
        q = torch.randn(n, nh, hd, generator=g)
        if craft:
            craft(r, q, k, v)
        k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
        for b in range(-(-total // page)):
            pg = perm.pop()
            tables[r, b] = pg
            m = min(page, total - b * page)
            kp[pg, :, :m] = k[b * page:b * page + m].transpose(0, 1)
            vp[pg, :, :m] = v[b * page:b * page + m].transpose(0, 1)
        if window:  # pages the window has passed for every query of the step are given back
            first_needed = max(0, c - window + 1)
            for b in range(width):
                if (b + 1) * page <= first_needed:
                    tables[r, b] = -1
        qs.append(q); ks.append(k); vs.append(v)
        segs.append((t0, n, c))
        t0 += n
    tile = ops.attention_tile_tokens(nh, nkv, dtype, hd, page, window or 0)
    # (splits from 128 keys on, shorter than the engine cuts them, so that the short contexts here have some)
    work, red, parts = attention_plan.plan_attention(segs, tile, window, nkv * (-(-(nh // nkv) // 16)), target_ctas,
                                                     min_split_keys=min_split_keys,
                                                     multi_min_split_keys=multi_min_split_keys)
    dev = lambda t: t.to(DEV)
    workd = dev(torch.from_numpy(np.ascontiguousarray(work)).reshape(-1, 8)) if len(work) else torch.zeros(1, 8, dtype=torch.int32, device=DEV)
    if idle_items:   # a list with room to spare, as a captured step's is
        workd = torch.cat([workd, torch.zeros(idle_items, 8, dtype=torch.int32, device=DEV)])
    redd = dev(torch.from_numpy(np.ascontiguousarray(red)).reshape(-1, 4)) if len(red) else torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    qd = dev(torch.cat(qs).reshape(t0, nh * hd).contiguous())
    out = torch.zeros_like(qd)
    part_o = torch.zeros(max(parts, 1), nh, hd, device=DEV)
    part_ml = torch.zeros(max(parts, 1), nh, 2, device=DEV)
    st = status()
    # the tensor-core kernels read pools whose rows are stored swizzled (as the cache-write kernel stores them)
    swz = ops.pool_is_swizzled(dtype, nh, nkv, hd)
    kpd, vpd = dev(kp), dev(vp)
    if swz:
        ops.swizzle_pool_(kpd); ops.swizzle_pool_(vpd)
    w = AttentionWork(workd, dev(torch.tensor([len(work)], dtype=torch.int32)), len(work) + idle_items, redd,
                      dev(torch.tensor([len(red)], dtype=torch.int32)), len(red), part_o, part_ml, kinds=kinds,
                      many_splits=attention_plan.many_splits(len(reqs), nkv * (-(-(nh // nkv) // 16)), target_ctas))
    ops.paged_attention(qd, kpd, vpd, dev(tables), w, out, nh, nkv, hd, window or 0, scale, st, swizzled=swz)
    assert st.item() == 0
    if raw:
        return out, len(red)
    res = []
    for (a, n, c), q, k, v in zip(segs, qs, ks, vs):
        want = attention_ref(q.float(), k.float(), v.float(), scale, window)
        res.append((out[a:a + n].view(n, nh, hd).double().cpu(), want))
    return res, len(red)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,page,window", [
    (6, 3, 48, 8, None), (8, 1, 32, 16, None), (16, 8, 128, 16, None), (4, 4, 80, 64, None),
    (32, 1, 16, 8, None), (8, 2, 64, 16, 40), (6, 3, 48, 8, 7), (2, 1, 256, 32, None),
    (4, 4, 128, 16, None), (8, 1, 64, 8, None), (9, 3, 128, 12, 50), (40, 2, 64, 16, None), (32, 8, 128, 64, None)])
def test_paged_attention_mixed_batch(dtype, nh, nkv, hd, page, window):
    # portions beside decoded tokens, contexts that end on and off page edges
    reqs = [(0, 1), (0, 37), (63, 1), (64, 1), (130, 2), (17, 50), (300, 1), (page * 3 - 1, 3)]
    for target in (1, 10 ** 6):     # never split / split wherever the range is long enough
        res, n_red = run_attention(dtype, reqs, nh, nkv, hd, page, window, target)
        assert (n_red > 0) == (target > 1 and not (window and window < 128))
        for got, want in res:
            torch.testing.assert_close(got, want, **tol(dtype))


@pytest.mark.parametrize("nh,nkv,hd,page", [(16, 8, 128, 16), (8, 1, 64, 8), (32, 8, 128, 64), (40, 2, 64, 16),
                                            (4, 4, 128, 128), (6, 3, 64, 32)])
def test_decode_only_steps_take_the_bulk_copy_kernel(nh, nkv, hd, page):
    # single decoded tokens: contexts that end on and off tile and page edges, one of a single key
    reqs = [(0, 1), (63, 1), (64, 1), (127, 1), (128, 1), (700, 1), (1023, 1), (15, 1), (page * 3, 1), (331, 1)]
    assert ops.lib().pllm_attention_decode_tma_supports(1, nh, nkv, hd, page, 0)
    for target in (1, 10 ** 6):
        res, n_red = run_attention(torch.bfloat16, reqs, nh, nkv, hd, page, None, target, kinds=1)
        assert (n_red > 0) == (target > 1)
        for got, want in res:
            torch.testing.assert_close(got, want, **tol(torch.bfloat16))
    # and beside portions of several tokens, where both kernels share one work list
    res, _ = run_attention(torch.bfloat16, [(100, 1), (40, 9), (513, 1), (0, 70)], nh, nkv, hd, page, None, 10 ** 6, kinds=3)
    for got, want in res:
        torch.testing.assert_close(got, want, **tol(torch.bfloat16))


@pytest.mark.parametrize("nh,nkv,hd,page", [(16, 8, 128, 16), (8, 1, 64, 8), (4, 4, 128, 64), (6, 3, 64, 32), (40, 2, 64, 16),
                                            (5, 1, 128, 16)])
def test_prompt_portions_take_the_tcgen05_kernel(monkeypatch, nh, nkv, hd, page):
    # portions of many tokens, with and without context before them, ending on and off the edges of
    # the 64-key tiles and of the 128-row items; beside single decoded tokens (which it then takes too)
    assert ops.attention_prefill_uses_tcgen05(torch.bfloat16, nh, nkv, hd, page, 0)
    reqs = [(0, 300), (1000, 200), (37, 129), (63, 2), (500, 1), (0, 64), (64, 65), (0, 1)]
    # the single tokens beside the portions: on the bulk-copy kernel on a second stream, or in the tcgen05 kernel too
    for beside, expect in ((True, 6), (False, 4)):
        monkeypatch.setattr(ops, "MIXED_BESIDE", beside)
        monkeypatch.setattr(ops, "MIXED_BESIDE_MIN_REQUESTS", 1)
        launches = ops.LAUNCHES
        for target in (1, 10 ** 6):
            res, _ = run_attention(torch.bfloat16, reqs, nh, nkv, hd, page, None, target)
            for got, want in res:
                torch.testing.assert_close(got, want, **tol(torch.bfloat16))
        assert ops.LAUNCHES - launches == expect     # (bulk copy +) tcgen05 + reduction, twice
    # one key far back decides the row: its score stands out, and its value is unlike the others
    def craft(r, q, k, v):
        if r == 0:
            q[250] *= 0; q[250, :, 3] = 16.0
            k[:, :, 3] = -1.0; k[41, :, 3] = 16.0
            v[41] = 5.0
    res, _ = run_attention(torch.bfloat16, [(0, 300)], nh, nkv, hd, page, None, 1, craft=craft)
    got, want = res[0]
    assert (got[250] - 5.0).abs().max() < 0.1
    torch.testing.assert_close(got, want, **tol(torch.bfloat16))


@pytest.mark.parametrize("nh,nkv,hd,page,norm,rope", [(16, 8, 128, 16, True, True), (8, 1, 64, 8, True, True),
                                                        (40, 2, 64, 16, False, True), (4, 4, 128, 64, True, False),
                                                        (6, 3, 64, 32, False, False)])
def test_decode_attention_does_the_norm_the_rotation_and_the_cache_write_itself(nh, nkv, hd, page, norm, rope):
    # the same decode step two ways: the q/k kernel then the attention kernels, and the attention
    # kernel alone from the projection's output.  Outputs and both pools must be equal bit for bit.
    from paged_llm_rs_b200.parts.base import Runtime
    from paged_llm_rs_b200.parts.position import RotaryEncoding
    from paged_llm_rs_b200.parts.spec import PartSpec
    assert ops.decode_attention_fuses(torch.bfloat16, nh, nkv, hd, page, 0, hd if rope else 0, True)
    g = torch.Generator(device=DEV).manual_seed(nh + hd)
    ctxs = [0, 1, 63, 64, 127, 700, 1023, 15, page * 3, 331, 2000]         # tokens in the cache before the step
    B = len(ctxs)
    width = max(-(-(c + 1) // page) for c in ctxs)
    n_pages = sum(-(-(c + 1) // page) for c in ctxs) + 2
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1)).tolist()
    tables = torch.full((B, width), -1, dtype=torch.int32)
    for r, c in enumerate(ctxs):
        for b in range(-(-(c + 1) // page)):
            tables[r, b] = perm.pop()
    tables = tables.to(DEV)
    kp = torch.randn(n_pages, nkv, page, hd, device=DEV, generator=g).bfloat16()
    vp = torch.randn(n_pages, nkv, page, hd, device=DEV, generator=g).bfloat16()
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, device=DEV, generator=g).bfloat16()
    qg = 1 + 0.1 * torch.randn(hd, device=DEV, generator=g) if norm else None
    kg = 1 + 0.1 * torch.randn(hd, device=DEV, generator=g) if norm else None
    cos = sin = None
    if rope:
        enc = RotaryEncoding(PartSpec("rope", dict(head_dim=hd, rotary_dim=hd, theta=1e6, max_positions=4096)),
                             Runtime(torch.device(DEV), torch.bfloat16))
        cos, sin, _ = enc.rotary()
    pos = torch.tensor(ctxs, dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(tables[r, c // page]) * page + c % page for r, c in enumerate(ctxs)], dtype=torch.int32, device=DEV)
    for target in (1, 10 ** 6):     # whole; split
        work, red, parts = attention_plan.plan_attention([(r, 1, c) for r, c in enumerate(ctxs)], 1, None, nkv * (-(-(nh // nkv) // 16)),
                                                         target, min_split_keys=128)
        workd = torch.from_numpy(np.ascontiguousarray(work)).reshape(-1, 8).to(DEV)
        redd = torch.from_numpy(np.ascontiguousarray(red)).reshape(-1, 4).to(DEV) if len(red) else torch.zeros(1, 4, dtype=torch.int32, device=DEV)
        nw = torch.tensor([len(work)], dtype=torch.int32, device=DEV)
        nr = torch.tensor([len(red)], dtype=torch.int32, device=DEV)
        part_o = torch.zeros(max(parts, 1), nh, hd, device=DEV)
        part_ml = torch.zeros(max(parts, 1), nh, 2, device=DEV)
        st = status()
        # the two kernels
        k1, v1 = kp.clone(), vp.clone()
        q = torch.empty(B, nh * hd, device=DEV, dtype=torch.bfloat16)
        ops.qk_norm_rope_kv(qkv, q, qg, kg, 1e-6, cos, sin, hd if rope else 0, pos, slots, k1, v1, nh, nkv, hd, st, swizzled=True)
        o1 = torch.zeros_like(q)
        w = AttentionWork(workd, nw, len(work), redd, nr, len(red), part_o, part_ml, kinds=1)
        ops.paged_attention(q, k1, v1, tables, w, o1, nh, nkv, hd, 0, hd ** -0.5, st, swizzled=True)
        # the one
        k2, v2 = kp.clone(), vp.clone()
        o2 = torch.zeros_like(q)
        ops.decode_attention_fused(qkv, qg, kg, 1e-6, cos, sin, k2, v2, tables, w, o2, nh, nkv, hd, hd ** -0.5, st)
        assert st.item() == 0
        assert torch.equal(k1, k2) and torch.equal(v1, v2)
        assert not torch.equal(k1, kp)                   # (the step did write)
        assert torch.equal(o1, o2)


def test_swizzled_cache_rows():
    from paged_llm_rs_b200.parts.base import Runtime
    g = torch.Generator(device=DEV).manual_seed(4)
    T, nh, nkv, hd, page, pages = 40, 4, 2, 128, 16, 5
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV, generator=g).bfloat16()
    pos = torch.arange(T, device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * page, device=DEV, generator=g)[:T].to(torch.int32)
    pools = {}
    for swz in (False, True):
        kp = torch.zeros(pages, nkv, page, hd, device=DEV, dtype=torch.bfloat16)
        vp = torch.zeros_like(kp)
        q = torch.empty(T, nh * hd, device=DEV, dtype=torch.bfloat16)
        ops.qk_norm_rope_kv(qkv, q, None, None, 0.0, None, None, 0, pos, slots, kp, vp, nh, nkv, hd, status(), swizzled=swz)
        pools[swz] = (kp, vp, q)
    assert torch.equal(pools[False][2], pools[True][2])                       # q is never swizzled
    assert not torch.equal(pools[False][0], pools[True][0])
    assert torch.equal(ops.swizzle_pool_(pools[False][0].clone()), pools[True][0])
    assert torch.equal(ops.swizzle_pool_(pools[False][1].clone()), pools[True][1])


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_decides(dtype):
    # One key early in a long context matches the query; its value is a marker.  A
    # kernel that loses that key (a wrong page, a range cut short) cannot return the marker.
    def craft(r, q, k, v):
        far = 3 + 5 * r
        k[far] = 0; k[far, :, 0] = 8.0
        q[:] = 0; q[:, :, 0] = 8.0 * (q.shape[-1] ** 0.5)
        v[far] = 100.0 + r
    reqs = [(700, 1), (517, 1), (333, 2)]
    for target in (1, 10 ** 6):
        res, _ = run_attention(dtype, reqs, 4, 2, 64, 16, None, target, craft=craft)
        for r, (got, want) in enumerate(res):
            assert (got - (100.0 + r)).abs().max() < 0.6
            torch.testing.assert_close(got, want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("context", [4096, 16384, 40000])
def test_a_far_key_decides_in_a_long_context(dtype, context):
    # The reference's kernel holds a score per key in shared memory and stops at 12 160 keys
    # (crates/pagedllm/src/kernels/paged_attention.rs:626-634); this one cuts the range into splits and
    # combines them.  Contexts up to the 0.6B shape's 40 960 positions, cut as the engine cuts them
    # (296 CTAs wanted, splits of at least 256 keys, up to 128 of them) and not cut at all: a key near
    # the start of the context carries the answer, and the very first and the very last key carry
    # louder wrong ones that the right one must still beat.
    nh, nkv, hd, page = 4, 1, 128, 16

    def craft(r, q, k, v):
        far = 70 + 300 * r
        q[:] = 0; q[:, :, 5] = 9.0 * hd ** 0.5
        k[:, :, 5] = 0
        k[far, :, 5] = 9.0; v[far] = 40.0 + r
        k[0, :, 5] = 7.0; v[0] = -200.0
        k[-1, :, 5] = 7.0; v[-1] = 300.0
    reqs = [(context - 1, 1), (context - 1 - 77, 1)]
    for target, splits in ((1, False), (296, True)):
        res, n_red = run_attention(dtype, reqs, nh, nkv, hd, page, None, target, craft=craft, kinds=1,
                                   min_split_keys=attention_plan.MIN_SPLIT_KEYS)
        assert (n_red > 0) == splits
        for r, (got, want) in enumerate(res):
            assert (got - (40.0 + r)).abs().max() < 1.0
            torch.testing.assert_close(got, want, **tol(dtype))


def test_a_far_key_decides_for_a_long_portion_behind_a_long_context():
    # 2048 tokens of a prompt behind 6000 that are already in the cache: the tcgen05 kernel's tiles of
    # 128 rows walk some 8000 keys through the block table; a key in the cached part decides for one
    # row, and one inside the portion for another
    nh, nkv, hd, page = 4, 1, 128, 16
    assert ops.attention_prefill_uses_tcgen05(torch.bfloat16, nh, nkv, hd, page, 0)

    def craft(r, q, k, v):
        k[:, :, 5] = 0
        for row, far, mark in ((1500, 41, 30.0), (77, 6000 + 500, -20.0), (2047, 5999, 11.0)):
            q[row] = 0; q[row, :, 5] = 9.0 * hd ** 0.5
            k[far, :, 5] = 9.0; v[far] = mark
    res, _ = run_attention(torch.bfloat16, [(6000, 2048)], nh, nkv, hd, page, None, 296, craft=craft, kinds=2,
                           min_split_keys=attention_plan.MIN_SPLIT_KEYS,
                           multi_min_split_keys=attention_plan.MULTI_MIN_SPLIT_KEYS)
    got, want = res[0]
    # row 77 (position 6077) sees the marked keys at 41 and 5999, which score alike: the mean of their
    # values; rows 1500 and 2047 see the one at 6500 too
    assert (got[77] - 20.5).abs().max() < 0.5
    assert (got[1500] - 7.0).abs().max() < 0.5 and (got[2047] - 7.0).abs().max() < 0.5
    torch.testing.assert_close(got, want, **tol(torch.bfloat16))


def test_a_short_portion_behind_thirty_thousand_tokens():
    # 130 tokens of a prompt behind 30 000 in the cache: each softmax group of the tcgen05 kernel walks
    # some 235 tiles of keys when the range is left whole (its barriers change phase hundreds of times), and
    # the tiles of several tokens are cut into splits whose partial rows the reduction combines when the
    # launch wants more CTAs.  A key near the start decides for one row; a later row also sees a marked key of the portion itself.
    nh, nkv, hd, page = 4, 1, 128, 16
    assert ops.attention_prefill_uses_tcgen05(torch.bfloat16, nh, nkv, hd, page, 0)

    def craft(r, q, k, v):
        k[:, :, 5] = 0
        for row, far, mark in ((3, 41, 30.0), (129, 30100, -20.0)):
            q[row] = 0; q[row, :, 5] = 9.0 * hd ** 0.5
            k[far, :, 5] = 9.0; v[far] = mark
    for target, splits in ((1, False), (296, True)):
        res, n_red = run_attention(torch.bfloat16, [(30000, 130)], nh, nkv, hd, page, None, target, craft=craft, kinds=2,
                                   min_split_keys=attention_plan.MIN_SPLIT_KEYS,
                                   multi_min_split_keys=attention_plan.MULTI_MIN_SPLIT_KEYS)
        assert (n_red > 0) == splits
        got, want = res[0]
        assert (got[3] - 30.0).abs().max() < 0.5            # position 30003 sees the marked key at 41 and not the one at 30100
        assert (got[129] - 5.0).abs().max() < 0.5           # position 30129 sees both marked keys, which score alike
        torch.testing.assert_close(got, want, **tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edge(dtype):
    # window 24: the query at position p sees keys p-23..p.  The key at p-23 carries the
    # answer; the key at p-24, just outside, carries a louder wrong one.
    W = 24

    def craft(r, q, k, v):
        p = k.shape[0] - 1
        q[:] = 0; q[:, :, 1] = 6.0 * (q.shape[-1] ** 0.5)
        k[:, :, 1] = 0
        k[p - W + 1, :, 1] = 6.0; v[p - W + 1] = 7.0
        k[p - W, :, 1] = 12.0; v[p - W] = -50.0
    res, _ = run_attention(dtype, [(90, 1), (47, 1), (24, 1)], 4, 2, 32, 8, W, 1, craft=craft)
    for got, want in res:
        assert (got - 7.0).abs().max() < 0.5
        torch.testing.assert_close(got, want, **tol(dtype))


def test_attention_refuses_sizes_it_does_not_take():
    from paged_llm_rs_b200.errors import KernelError
    with pytest.raises(KernelError, match="head_dim"):
        run_attention(torch.float32, [(3, 1)], 2, 1, 24, 8, None, 1)
    with pytest.raises(KernelError, match="head_dim"):
        run_attention(torch.float32, [(3, 1)], 2, 1, 512, 8, None, 1)


def test_kernels_refuse_host_tensors():
    from paged_llm_rs_b200.errors import KernelError
    with pytest.raises(KernelError, match="no CPU path"):
        ops.swiglu(torch.zeros(2, 8), torch.zeros(2, 4))


# --- sampling ----------------------------------------------------------------------------

@pytest.mark.parametrize("vocab", [1000, 151936, 33])
def test_sampling_kernel(vocab):
    g = torch.Generator(device=DEV).manual_seed(5)
    n = 24
    logits = torch.randn(n, vocab, device=DEV, generator=g) * 4
    logits[0, 7] = logits[0, 3] = 99.0              # a tie: the first maximum wins
    temp = torch.zeros(n, device=DEV)
    temp[n // 2:] = torch.rand(n - n // 2, device=DEV, generator=g) + 0.3
    u = torch.rand(n, device=DEV, generator=g)
    u[n // 2] = 0.0
    toks = torch.zeros(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, temp, u, toks)
    toks = toks.cpu().tolist()
    lg = logits.cpu().double()
    assert toks[0] == 3
    for i in range(n // 2):
        assert toks[i] == int(lg[i].argmax())
    for i in range(n // 2, n):
        p = torch.softmax(lg[i] / temp[i].item(), -1)
        cdf = torch.cumsum(p, 0)
        point = u[i].item()
        # the token whose span of the running sum holds the point, give or take float32 rounding
        lo = cdf[toks[i] - 1].item() if toks[i] > 0 else 0.0
        assert lo - 1e-4 <= point <= cdf[toks[i]].item() + 1e-4, i


@pytest.mark.parametrize("M", [1, 3, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K", [(1024, 2048), (6144, 1024), (304, 384), (151936, 128), (48, 3072)])
def test_skinny_gemm(M, N, K):
    g = torch.Generator(device=DEV).manual_seed(M * 1000 + N)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    ops.SKINNY_MAX_M = 64
    assert ops.skinny_gemm_takes(x, w)
    ops.SKINNY_MAX_N, ops.SKINNY_MAX_M = 1 << 20, 64      # here also the widest and tallest shapes go through the kernel
    want = x.float() @ w.float().T
    torch.testing.assert_close(ops.linear(x, w).float(), want, atol=2e-2, rtol=2e-2)
    y32 = ops.linear(x, w, out_dtype=torch.float32)
    assert y32.dtype == torch.float32
    torch.testing.assert_close(y32, want, atol=2e-3, rtol=2e-3)      # float accumulation, no bfloat16 rounding of the sum
    # the gated form: silu(g) * u on the way in
    gu = torch.randn(M, 2 * K, device=DEV, generator=g).bfloat16()
    a = gu.float()[:, :K]
    act = (a * torch.sigmoid(a) * gu.float()[:, K:]).bfloat16().float()
    torch.testing.assert_close(ops.linear(gu, w, gated=True).float(), act @ w.float().T, atol=3e-2, rtol=3e-2)
    ops.SKINNY_MAX_N, ops.SKINNY_MAX_M = 32768, 16


def _rms_ref(h, gain, eps):
    return h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * gain


@pytest.mark.parametrize("M", [1, 7, 16])
@pytest.mark.parametrize("I,K", [(3072, 1024), (304, 384), (16, 128), (1000, 256), (12288, 4096)])
def test_gate_and_up_product_with_the_activation_folded_in(M, I, K):
    g = torch.Generator(device=DEV).manual_seed(M * 31 + I + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV, generator=g) * 0.05).bfloat16()
    gu = (x.float() @ w.float().T).bfloat16().float()
    want = gu[:, :I] * torch.sigmoid(gu[:, :I]) * gu[:, I:]
    launches = ops.LAUNCHES
    y = ops.linear_glu(x, w)
    if I % 16 == 0:
        assert ops.skinny_glu_takes(x, w, I) and ops.LAUNCHES - launches == 1     # both products and the activation: one kernel
    assert y.shape == (M, I)
    torch.testing.assert_close(y.float(), want, atol=2e-2, rtol=3e-2)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (1, 128, 64), (77, 256, 1024), (200, 384, 72), (300, 512, 320),
                                   (2048, 4096, 1024), (640, 1024, 2048), (129, 1280, 136)])
def test_tcgen05_product(M, N, K):
    # tiles of 128 x 128 and 128 x 256, rows and k that end off a tile's edge, several tiles a CTA
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    st = status()
    y = ops.gemm_tcgen05(x, w, status=st)
    assert st.item() == 0 and y.shape == (M, N) and y.dtype == torch.bfloat16
    torch.testing.assert_close(y.float(), x.float() @ w.float().T, atol=3e-2, rtol=2e-2)
    # one far entry of W decides a column: a wrong k block or swizzle would lose it
    w2 = w.clone(); w2[N - 1, K - 1] = 100.0
    y2 = ops.gemm_tcgen05(x, w2, status=st)
    torch.testing.assert_close(y2.float()[:, N - 1], (x.float() @ w2.float().T)[:, N - 1], atol=0.5, rtol=2e-2)
    assert torch.equal(y2[:, :N - 1], y[:, :N - 1])


@pytest.mark.parametrize("M,I,K", [(128, 64, 64), (5, 64, 128), (300, 192, 320), (2048, 3072, 1024), (200, 640, 72)])
def test_tcgen05_product_with_the_gated_activation(M, I, K):
    g = torch.Generator(device=DEV).manual_seed(M + I + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV, generator=g) * 0.05).bfloat16()
    st = status()
    y = ops.gemm_tcgen05(x, w, glu=True, status=st)
    assert st.item() == 0 and y.shape == (M, I)
    gu = (x.float() @ w.float().T).bfloat16().float()
    want = gu[:, :I] * torch.sigmoid(gu[:, :I]) * gu[:, I:]
    # gate and up are rounded to bfloat16 before the activation on both sides; sums that differ in
    # the last place flip a rounding now and then, which the activation scales by the other factor
    scale = 1 + gu[:, :I].abs() + gu[:, I:].abs()
    assert ((y.float() - want).abs() / scale).max().item() < 2e-2
    # the engine's route for a prompt portion gives the same
    was, ops.TCGEN05_GEMM = ops.TCGEN05_GEMM, 1
    try:
        if M >= ops.TCGEN05_MIN_M:
            assert torch.equal(ops.linear_glu(x, w, status=st), y)
    finally:
        ops.TCGEN05_GEMM = was
    ops.TCGEN05_GEMM = 0
    try:
        lib_route = ops.linear_glu(x, w)
    finally:
        ops.TCGEN05_GEMM = was
    assert ((y.float() - lib_route.float()).abs() / scale).max().item() < 2e-2


def test_linear_falls_back_to_the_library_for_other_shapes():
    g = torch.Generator(device=DEV).manual_seed(0)
    for M, N, K, dt in ((100, 256, 256, torch.bfloat16), (4, 250, 256, torch.bfloat16), (4, 256, 200, torch.bfloat16),
                        (4, 256, 256, torch.float32)):
        x = torch.randn(M, K, device=DEV, generator=g).to(dt)
        w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).to(dt)
        assert not ops.skinny_gemm_takes(x, w)
        t = dict(atol=2e-2, rtol=2e-2) if dt == torch.bfloat16 else dict(atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(ops.linear(x, w).float(), x.float() @ w.float().T, **t)
        gu = torch.randn(M, 2 * K, device=DEV, generator=g).to(dt)
        a = gu.float()[:, :K]
        act = (a * torch.sigmoid(a) * gu.float()[:, K:]).to(dt).float()
        torch.testing.assert_close(ops.linear(gu, w, gated=True).float(), act @ w.float().T, **t)


def test_sampling_kernel_follows_the_distribution():
    probs = torch.tensor([0.5, 0.3, 0.15, 0.05])
    n = 4000
    logits = torch.log(probs).repeat(n, 1).to(DEV).contiguous()
    u = torch.rand(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(9))
    toks = torch.zeros(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, torch.ones(n, device=DEV), u, toks)
    freq = torch.bincount(toks.long().cpu(), minlength=4).double() / n
    assert (freq - probs.double()).abs().max() < 0.03
