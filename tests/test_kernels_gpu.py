"""Each kernel alone against a plain 32-bit reference of the same op, at sizes other than the
engine's (odd ones, as tiny-llm's own tests use: 107, 127, 241, 255, 353)."""
import math
import types

import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == "float32" else 2.0 ** -7) * scale


@pytest.fixture(scope="module")
def ops():
    from tiny_llm_b200 import ops
    return ops


@pytest.mark.parametrize("dtype", DT)
def test_embedding(ops, dtype):
    torch.manual_seed(0)
    table = torch.randn(331, 241).to(DT[dtype])
    toks = torch.randint(0, 331, (57,), dtype=torch.int32)
    out = torch.empty(57, 241, device=DEV)
    ops.embedding(toks.to(DEV), table.to(DEV), out)
    assert torch.equal(out.cpu(), pl.embedding(table.float(), toks))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("rows,width,eps", [(107, 241, 1.192e-7), (5, 4096 + 48, 1e-5), (3, 16, 1e-6)])
def test_rms_norm(ops, dtype, rows, width, eps):
    torch.manual_seed(1)
    x = torch.randn(rows, width) * 3
    w = torch.randn(width)
    out = torch.empty(rows, width, dtype=DT[dtype], device=DEV)
    ops.rms_norm(x.to(DEV), w.to(DEV), eps, out)
    ref = pl.rms_norm(x, w, eps)
    assert float((out.float().cpu() - ref).abs().max()) <= tol(dtype, float(ref.abs().max()))
    pick = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32)
    out2 = torch.empty(3, width, dtype=DT[dtype], device=DEV)
    ops.rms_norm(x.to(DEV), w.to(DEV), eps, out2, pick.to(DEV))
    assert torch.equal(out2.cpu(), out.cpu()[pick.long()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("m,n,k", [(127, 353, 255), (1, 331, 80), (64, 64, 16), (200, 40, 1000), (3, 2, 1),
                                   (8, 640, 1024), (300, 520, 328), (129, 256, 72)])
def test_linear(ops, dtype, m, n, k):
    torch.manual_seed(2)
    a = torch.randn(m, k).to(DT[dtype])
    w = torch.randn(n, k).to(DT[dtype])
    ref = pl.linear(a.float().double(), w.float().double()).float()
    scale = float(ref.abs().max())
    same = torch.empty(m, n, dtype=DT[dtype], device=DEV)
    ops.linear(a.to(DEV), w.to(DEV), same)
    assert float((same.float().cpu() - ref).abs().max()) <= tol(dtype, scale)
    f32 = torch.empty(m, n, device=DEV)
    ops.linear(a.to(DEV), w.to(DEV), f32)
    assert float((f32.cpu() - ref).abs().max()) <= 2e-5 * max(scale, 1)    # 32-bit accumulation in both paths
    acc = torch.full((m, n), 0.5, device=DEV)
    ops.linear(a.to(DEV), w.to(DEV), acc, accumulate=True)
    assert float((acc.cpu() - ref - 0.5).abs().max()) <= 2e-5 * max(scale, 1)
    # a strided input (rows of a wider buffer) and a row's result that does not depend on its batch
    wide = torch.randn(m, k + 24).to(DT[dtype]).to(DEV)
    wide[:, :k] = a.to(DEV)
    out2 = torch.empty(m, n, device=DEV)
    ops.linear(wide[:, :k], w.to(DEV), out2)
    assert torch.equal(out2, f32)
    one = torch.empty(1, n, device=DEV)
    ops.linear(a[m // 2: m // 2 + 1].to(DEV), w.to(DEV), one)
    if dtype == "float32":
        assert torch.equal(one[0], f32[m // 2])                  # the 32-bit path orders its sums by k only
    else:
        assert float((one[0] - f32[m // 2]).abs().max()) <= 2e-5 * max(scale, 1)
    ops.check_status()


@pytest.mark.parametrize("m,n,k", [(1, 2048, 2048), (2, 37, 132), (3, 640, 5632), (4, 16, 4), (5, 331, 80), (8, 2560, 2048),
                                   (9, 250, 1000), (16, 24, 388), (13, 7, 128),
                                   (300, 520, 328), (2048, 256, 2048), (129, 130, 72), (128, 128, 4)])
def test_float32_linear_of_few_rows_gives_the_bits_of_the_tile_kernel(ops, m, n, k, monkeypatch):
    """Up to 16 float32 rows run on a kernel of their own, products of at least 128 x 128 on 128 x 128 tiles; every
    output element is the same chain of fmaf over ascending k as in the 64 x 64 tiles, so all agree to the bit, for
    every row count, for widths and depths that fill no tile or chunk, for a strided input and when adding into the
    output."""
    torch.manual_seed(m * 1000 + n)
    a = torch.randn(m, k + 8, device=DEV)[:, :k]
    w = torch.randn(n, k, device=DEV)
    ref = pl.linear(a.double().cpu(), w.double().cpu()).float()
    outs = []
    for skinny in (True, False):
        monkeypatch.setattr(ops, "linear_skinny", skinny)
        out = torch.empty(m, n + 4, device=DEV)[:, :n]
        ops.linear(a, w, out)
        acc = torch.full((m, n), 0.25, device=DEV)
        ops.linear(a, w, acc, accumulate=True)
        outs.append((out.clone(), acc))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    scale = max(1.0, float(ref.abs().max()))
    assert float((outs[0][0].cpu() - ref).abs().max()) <= 2e-5 * scale
    assert float((outs[0][1].cpu() - ref - 0.25).abs().max()) <= 2e-5 * scale
    ops.check_status()


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("m,inter,block", [(37, 176, 16), (5, 208, 16), (3, 5632, 128), (9, 7, 1)])
def test_silu_mul(ops, dtype, m, inter, block):
    from tiny_llm_b200.parts import interleave_gate_up
    torch.manual_seed(3)
    gate, up = torch.randn(m, inter).to(DT[dtype]), torch.randn(m, inter).to(DT[dtype])
    gu = interleave_gate_up(gate.t().contiguous(), up.t().contiguous(), block).t().contiguous()   # columns interleaved
    out = torch.empty(m, inter, dtype=DT[dtype], device=DEV)
    ops.silu_mul(gu.to(DEV), out, block)
    ref = pl.silu(gate.float()) * up.float()
    assert float((out.float().cpu() - ref).abs().max()) <= tol(dtype, float(ref.abs().max()))
    if dtype == "bfloat16":   # a float32 accumulation buffer as the source: same result, buffer handed back zeroed
        acc = gu.float().to(DEV)
        out2 = torch.empty_like(out)
        ops.silu_mul(acc, out2, block, consume=True)
        assert torch.equal(out2, out) and float(acc.abs().sum()) == 0.0


@pytest.mark.parametrize("m,n,k", [(8, 640, 1024), (1, 2048, 2048), (40, 384, 1536), (100, 200, 4096), (16, 128, 512)])
def test_linear_with_k_slices_reduced_in_a_cluster(ops, m, n, k, monkeypatch):
    """Few rows and a long K: the slices of K of a weight tile meet in a thread-block cluster (an option
    for the plain products, whose default is float32 atomics).  Sums are exact to 32-bit accuracy, and
    two runs give the same bits (one writer per element, fixed order)."""
    monkeypatch.setattr(ops, "cluster_mask", 7)
    torch.manual_seed(12)
    a = torch.randn(m, k).to(torch.bfloat16)
    w = torch.randn(n, k).to(torch.bfloat16)
    assert ops._cluster_slices(n, k) > 1
    ref = pl.linear(a.float().double(), w.float().double()).float()
    scale = float(ref.abs().max())
    runs = []
    for _ in range(2):
        acc = torch.full((m, n), 0.25, device=DEV)
        ops.linear(a.to(DEV), w.to(DEV), acc, accumulate=True)
        runs.append(acc.cpu())
    assert float((runs[0] - ref - 0.25).abs().max()) <= 2e-5 * max(scale, 1)
    assert torch.equal(runs[0], runs[1])
    same = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.linear(a.to(DEV), w.to(DEV), same)
    assert float((same.float().cpu() - ref).abs().max()) <= tol("bfloat16", scale)
    for slices in (3, 7):   # cluster extents that do not divide the tile's 128 rows
        if slices <= -(-k // 64):
            acc = torch.full((m, n), 0.25, device=DEV)
            ops._cluster_call(ops.EPI_CL_ADD_F32, a.to(DEV), w.to(DEV), acc, slices)
            assert float((acc.cpu() - ref - 0.25).abs().max()) <= 2e-5 * max(scale, 1), slices
    ops.check_status()


@pytest.mark.parametrize("m,nq,nkv,hd,k,page", [(7, 6, 3, 32, 1024, 8), (1, 32, 4, 64, 2048, 16), (33, 2, 2, 128, 512, 4),
                                              (5, 5, 1, 16, 80, 8), (300, 6, 3, 64, 1024, 16), (257, 3, 1, 128, 328, 8),
                                              (2048, 32, 4, 64, 136, 16)])   # 160 tiles: the last round runs as strips
def test_qkv_projection_with_rotation_and_cache_write_in_its_epilogue(ops, m, nq, nkv, hd, k, page):
    torch.manual_seed(13)
    n_pages, max_pos = -(-m // page) + 6, 91
    cos, sin = pl.rope_tables(max_pos, hd, 5000.0)
    h = torch.randn(m, k).to(torch.bfloat16)
    w = (torch.randn((nq + 2 * nkv) * hd, k) / math.sqrt(k)).to(torch.bfloat16)
    pos = torch.randint(0, max_pos, (m,), dtype=torch.int32)
    slots = torch.randperm(n_pages * page)[:m].to(torch.int32)
    kc = torch.zeros(n_pages, nkv, page, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    qkv = torch.full((m, (nq + 2 * nkv) * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    assert ops.linear_rope_kv(h.to(DEV), w.to(DEV), qkv, pos.to(DEV), cos.to(DEV), sin.to(DEV), nq, nkv, hd, kc, vc,
                              slots.to(DEV))
    ops.check_status()
    proj = pl.bf16_quant(pl.linear(h.float(), w.float()))
    q_ref = pl.apply_rope(proj[:, : nq * hd].view(m, nq, hd), cos, sin, pos)
    k_ref = pl.apply_rope(proj[:, nq * hd: (nq + nkv) * hd].view(m, nkv, hd), cos, sin, pos)
    v_ref = proj[:, (nq + nkv) * hd:].view(m, nkv, hd)
    e = tol("bfloat16", 4.0)
    assert float((qkv[:, : nq * hd].float().cpu().view(m, nq, hd) - q_ref).abs().max()) <= e
    assert float((qkv[:, nq * hd:].float().cpu() - 7.0).abs().max()) == 0     # the rest of the row is not written
    kc, vc = kc.cpu(), vc.cpu()
    for i in range(m):
        pg, off = int(slots[i]) // page, int(slots[i]) % page
        assert float((kc[pg, :, off].float() - k_ref[i]).abs().max()) <= e
        assert float((vc[pg, :, off].float() - v_ref[i]).abs().max()) <= e
    written = torch.zeros(n_pages * page, dtype=torch.bool)
    written[slots.long()] = True
    assert float(kc.permute(0, 2, 1, 3).reshape(n_pages * page, -1)[~written].abs().sum()) == 0   # nothing else touched
    # queries only (a layer that reads another layer's cache), no rotation
    q_only = torch.empty(m, nq * hd, dtype=torch.bfloat16, device=DEV)
    assert ops.linear_rope_kv(h.to(DEV), w[: nq * hd].contiguous().to(DEV), q_only, pos.to(DEV), None, None, nq, nkv, hd,
                              None, None, None)
    assert float((q_only.float().cpu() - proj[:, : nq * hd]).abs().max()) <= e


def test_qkv_epilogue_declines_head_sizes_that_do_not_tile(ops):
    h = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(3 * 48, 64, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(4, 3 * 48, dtype=torch.bfloat16, device=DEV)
    pos = torch.zeros(4, dtype=torch.int32, device=DEV)
    assert not ops.linear_rope_kv(h, w, out, pos, None, None, 1, 1, 48, None, None, None)


@pytest.mark.parametrize("m,inter,k", [(8, 5632, 2048), (3, 256, 64), (70, 384, 1024)])
def test_swiglu_projection_in_a_cluster(ops, m, inter, k):
    """Gate tile, up tile and their K slices as one cluster, SiLU * up in the epilogue."""
    from tiny_llm_b200.engine import Workspace
    from tiny_llm_b200.parts import interleave_gate_up
    torch.manual_seed(14)
    a = torch.randn(m, k).to(torch.bfloat16)
    wg = (torch.randn(inter, k) / math.sqrt(k)).to(torch.bfloat16)
    wu = (torch.randn(inter, k) / math.sqrt(k)).to(torch.bfloat16)
    out = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(a.to(DEV), interleave_gate_up(wg, wu, 128).to(DEV), out, 128, Workspace(DEV))
    ops.check_status()
    ref = pl.silu(pl.linear(a.float(), wg.float())) * pl.linear(a.float(), wu.float())
    assert float((out.float().cpu() - ref).abs().max()) <= tol("bfloat16", max(1.0, float(ref.abs().max())))


def paged_setup(dtype, n_req, lens, nkv, hd, page, seed, spare_pages=3):
    """Random keys/values for n_req sequences scattered over shuffled pages; unwritten slots are NaN."""
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-l // page) for l in lens]
    n_pages = sum(blocks) + spare_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_blocks = max(blocks) + 2
    table = torch.full((n_req, max_blocks), -1, dtype=torch.int32)
    k_cache = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=DT[dtype])
    v_cache = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=DT[dtype])
    ks, vs = [], []
    for r, l in enumerate(lens):
        k = torch.randn(l, nkv, hd, generator=g).to(DT[dtype])
        v = torch.randn(l, nkv, hd, generator=g).to(DT[dtype])
        ks.append(k), vs.append(v)
        for b in range(blocks[r]):
            pg = perm.pop()
            table[r, b] = pg
            n = min(page, l - b * page)
            k_cache[pg, :, :n] = k[b * page: b * page + n].permute(1, 0, 2)
            v_cache[pg, :, :n] = v[b * page: b * page + n].permute(1, 0, 2)
    return table, k_cache, v_cache, ks, vs


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nq,nkv,hd,page,window", [(6, 3, 48, 8, None), (4, 1, 80, 16, None), (5, 5, 128, 32, None),
                                                    (2, 2, 256, 4, None), (8, 2, 16, 16, 37), (3, 1, 64, 8, 8)])
def test_paged_attention(ops, dtype, nq, nkv, hd, page, window):
    """Queries at the end of sequences of different lengths: some portions, some single tokens."""
    lens = [301, 64, 7, 130]
    q_lens = [5, 1, 7, 33]
    table, k_cache, v_cache, ks, vs = paged_setup(dtype, 4, lens, nkv, hd, page, seed=nq * hd)
    g = torch.Generator().manual_seed(7)
    t = sum(q_lens)
    width = (nq + 2 * nkv) * hd
    qkv = torch.randn(t, width, generator=g).to(DT[dtype])
    # a far key among hundreds: request 0's first query and its key 3 are scaled so that this score stands out
    qkv[0, :hd] *= 6.0
    ks[0][3, 0] = (qkv[0, :hd] / qkv[0, :hd].float().norm() * 8.0).to(DT[dtype])
    pg = int(table[0, 0])
    k_cache[pg, 0, 3] = ks[0][3, 0]
    tok_req = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(q_lens)])
    pos = torch.cat([torch.arange(l - n, l, dtype=torch.int32) for l, n in zip(lens, q_lens)])
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    starts = torch.tensor([l - n for l, n in zip(lens, q_lens)], dtype=torch.int32)
    batch = types.SimpleNamespace(token_request=tok_req.to(DEV), positions=pos.to(DEV), cu_q=cu.to(DEV),
                                  q_start=starts.to(DEV), num_requests=4, max_q_len=max(q_lens), max_kv_len=max(lens))
    out = torch.empty(t, nq * hd, dtype=DT[dtype], device=DEV)
    scale = 1.0 / math.sqrt(hd)
    from tiny_llm_b200.engine import Workspace
    ops.paged_attention(qkv.to(DEV), nq, nkv, hd, k_cache.to(DEV), v_cache.to(DEV), table.to(DEV), batch, out,
                        scale, window, Workspace(DEV))
    out = out.float().cpu()
    assert not torch.isnan(out).any()
    cur = 0
    for r, (l, n) in enumerate(zip(lens, q_lens)):
        q = qkv[cur: cur + n, : nq * hd].float().view(n, nq, hd)
        ref = pl.attention(q, ks[r].float(), vs[r].float(), pos[cur: cur + n], window=window).reshape(n, nq * hd)
        d = float((out[cur: cur + n] - ref).abs().max())
        assert d <= tol(dtype, max(1.0, float(ref.abs().max()))), (r, d)
        cur += n
    if window is None:   # the far key carries the first query's first head
        p = torch.softmax((qkv[0, :hd].float() * scale) @ ks[0][:lens[0] - q_lens[0] + 1, 0].float().t(), 0)
        assert float(p[3]) > 0.9


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("window", [None, 300])
@pytest.mark.parametrize("nq,nkv,hd", [(6, 2, 48), (8, 1, 64), (4, 4, 128), (10, 2, 256)])
def test_attention_of_the_32_bit_path_gives_the_same_bits_with_one_warp_or_eight_per_head(ops, dtype, window, nq, nkv, hd,
                                                                                           monkeypatch):
    """The kernel of the 32-bit path walks the keys as eight interleaved running softmaxes that are merged in a fixed
    order; with few (token, head) pairs eight warps carry one each, with many one warp walks them one after the other
    for up to four heads of a group at once (or, the plainest form, carries all eight for one head).  All must
    agree with the plain implementation and with each other to the bit, at contexts of a few tiles and of dozens, with
    a window and without: else a token's logits would depend on how many others shared its step."""
    from tiny_llm_b200.engine import Workspace
    page = 8
    lens, q_lens = [2100, 700, 33, 9], [1, 3, 2, 9]
    table, k_cache, v_cache, ks, vs = paged_setup(dtype, 4, lens, nkv, hd, page, seed=5)
    g = torch.Generator().manual_seed(3)
    t = sum(q_lens)
    qkv = torch.randn(t, (nq + 2 * nkv) * hd, generator=g).to(DT[dtype])
    tok_req = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(q_lens)])
    pos = torch.cat([torch.arange(l - n, l, dtype=torch.int32) for l, n in zip(lens, q_lens)])
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    starts = torch.tensor([l - n for l, n in zip(lens, q_lens)], dtype=torch.int32)
    batch = types.SimpleNamespace(token_request=tok_req.to(DEV), positions=pos.to(DEV), cu_q=cu.to(DEV),
                                  q_start=starts.to(DEV), num_requests=4, max_q_len=max(q_lens), max_kv_len=max(lens))
    monkeypatch.setattr(ops, "force_generic", True)
    outs = []
    for split in (False, True, 2):    # a warp per (token, kv head, four heads); eight warps per pair; one warp per pair
        monkeypatch.setattr(ops, "generic_attention_split", split)
        out = torch.empty(t, nq * hd, dtype=DT[dtype], device=DEV)
        ops.paged_attention(qkv.to(DEV), nq, nkv, hd, k_cache.to(DEV), v_cache.to(DEV), table.to(DEV), batch, out,
                            1.0 / math.sqrt(hd), window, Workspace(DEV))
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    cur = 0
    for r, (l, n) in enumerate(zip(lens, q_lens)):
        q = qkv[cur: cur + n, : nq * hd].float().view(n, nq, hd)
        ref = pl.attention(q, ks[r].float(), vs[r].float(), pos[cur: cur + n], window=window).reshape(n, nq * hd)
        d = float((outs[0][cur: cur + n].float() - ref).abs().max())
        assert d <= tol(dtype, max(1.0, float(ref.abs().max()))), (r, d)
        cur += n


@pytest.mark.parametrize("hd,nq,nkv,page", [(64, 8, 1, 16), (64, 32, 4, 16), (64, 4, 4, 8), (64, 2, 1, 64), (64, 16, 2, 32),
                                            (128, 8, 8, 16), (128, 32, 8, 16), (128, 4, 1, 8), (128, 2, 2, 64), (128, 16, 1, 32)])
def test_paged_attention_on_tcgen05(ops, hd, nq, nkv, page):
    """Head size 64 or 128 and portions of at least 128 rows: the tcgen05 kernel.  Portions that start in
    the middle of a sequence, end in the middle of a page, and a one-token request beside them; unwritten
    slots of the pages are NaN."""
    dtype = "bfloat16"
    lens = [700, 300, 129, 64]
    q_lens = [389, 300, 17, 1]
    table, k_cache, v_cache, ks, vs = paged_setup(dtype, 4, lens, nkv, hd, page, seed=nq + page)
    g = torch.Generator().manual_seed(8)
    t = sum(q_lens)
    width = (nq + 2 * nkv) * hd
    qkv = torch.randn(t, width, generator=g).to(DT[dtype])
    # a far key among hundreds: request 0's last query and its key 5 are scaled so that this score stands out
    last = q_lens[0] - 1
    qkv[last, :hd] *= 6.0
    ks[0][5, 0] = (qkv[last, :hd] / qkv[last, :hd].float().norm() * 8.0).to(DT[dtype])
    k_cache[int(table[0, 5 // page]), 0, 5 % page] = ks[0][5, 0]
    # ... and the query before it with key 450, eight tiles into the keys: the running maximum of that row jumps
    # far after O already holds seven tiles (the kernel rescales O only on such jumps)
    qkv[last - 1, :hd] *= 6.0
    ks[0][450, 0] = (qkv[last - 1, :hd] / qkv[last - 1, :hd].float().norm() * 8.0).to(DT[dtype])
    k_cache[int(table[0, 450 // page]), 0, 450 % page] = ks[0][450, 0]
    pos = torch.cat([torch.arange(l - n, l, dtype=torch.int32) for l, n in zip(lens, q_lens)])
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    starts = torch.tensor([l - n for l, n in zip(lens, q_lens)], dtype=torch.int32)
    tok_req = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(q_lens)])
    batch = types.SimpleNamespace(token_request=tok_req.to(DEV), positions=pos.to(DEV), cu_q=cu.to(DEV),
                                  q_start=starts.to(DEV), num_requests=4, max_q_len=max(q_lens), max_kv_len=max(lens))
    out = torch.full((t, nq * hd), float("nan"), dtype=DT[dtype], device=DEV)
    scale = 1.0 / math.sqrt(hd)
    from tiny_llm_b200 import ops as ops_mod
    from tiny_llm_b200.engine import Workspace
    before = set(ops_mod.build.loaded_libraries())
    ops.paged_attention(qkv.to(DEV), nq, nkv, hd, k_cache.to(DEV), v_cache.to(DEV), table.to(DEV), batch, out,
                        scale, None, Workspace(DEV))
    ops.check_status()
    assert f"attention_tc_head_dim{hd}" in set(ops_mod.build.loaded_libraries()) | before
    out = out.float().cpu()
    assert not torch.isnan(out).any()
    cur = 0
    for r, (l, n) in enumerate(zip(lens, q_lens)):
        q = qkv[cur: cur + n, : nq * hd].float().view(n, nq, hd)
        ref = pl.attention(q, ks[r].float(), vs[r].float(), pos[cur: cur + n], quant=pl.bf16_quant).reshape(n, nq * hd)
        d = float((out[cur: cur + n] - ref).abs().max())
        assert d <= tol(dtype, max(1.0, float(ref.abs().max()))), (r, d)
        cur += n
    p = torch.softmax((qkv[last, :hd].float() * scale) @ ks[0][:lens[0], 0].float().t(), 0)
    assert float(p[5]) > 0.9
    p = torch.softmax((qkv[last - 1, :hd].float() * scale) @ ks[0][:lens[0] - 1, 0].float().t(), 0)
    assert float(p[450]) > 0.9


@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("hd,nq,nkv,page", [(64, 32, 4, 16), (128, 8, 2, 32), (64, 4, 4, 8)])
def test_attention_of_decoded_tokens_beside_portions(ops, hd, nq, nkv, page, split, monkeypatch):
    """A step as the scheduler lays it out: requests with one token first, then portions.  The decoded tokens run on
    the decode kernel and the portions on the tcgen05 kernel, as two launches over two runs of the same tables
    (`split`), or all of them on the tcgen05 kernel; both against the plain implementation."""
    from tiny_llm_b200.engine import Workspace
    monkeypatch.setattr(ops, "split_mixed_attention", split)
    dtype = "bfloat16"
    lens = [1500, 1, 333, 64, 700, 300, 40]
    q_lens = [1, 1, 1, 1, 389, 300, 17]
    n_req = len(lens)
    table, k_cache, v_cache, ks, vs = paged_setup(dtype, n_req, lens, nkv, hd, page, seed=nq + page + 1)
    g = torch.Generator().manual_seed(18)
    t = sum(q_lens)
    qkv = torch.randn(t, (nq + 2 * nkv) * hd, generator=g).to(DT[dtype])
    # a far key among 1,500 for the first decoded token
    qkv[0, :hd] *= 6.0
    ks[0][77, 0] = (qkv[0, :hd] / qkv[0, :hd].float().norm() * 8.0).to(DT[dtype])
    k_cache[int(table[0, 77 // page]), 0, 77 % page] = ks[0][77, 0]
    pos = torch.cat([torch.arange(l - n, l, dtype=torch.int32) for l, n in zip(lens, q_lens)])
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    starts = torch.tensor([l - n for l, n in zip(lens, q_lens)], dtype=torch.int32)
    tok_req = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(q_lens)])
    batch = types.SimpleNamespace(token_request=tok_req.to(DEV), positions=pos.to(DEV), cu_q=cu.to(DEV),
                                  q_start=starts.to(DEV), num_requests=n_req, max_q_len=max(q_lens), max_kv_len=2048,
                                  num_leading_decodes=4)
    out = torch.full((t, nq * hd), float("nan"), dtype=DT[dtype], device=DEV)
    scale = 1.0 / math.sqrt(hd)
    before = ops.launches
    ops.paged_attention(qkv.to(DEV), nq, nkv, hd, k_cache.to(DEV), v_cache.to(DEV), table.to(DEV), batch, out,
                        scale, None, Workspace(DEV))
    ops.check_status()
    assert ops.launches - before == (2 if split else 1)
    out = out.float().cpu()
    assert not torch.isnan(out).any()
    cur = 0
    for r, (l, n) in enumerate(zip(lens, q_lens)):
        q = qkv[cur: cur + n, : nq * hd].float().view(n, nq, hd)
        ref = pl.attention(q, ks[r].float(), vs[r].float(), pos[cur: cur + n], quant=pl.bf16_quant).reshape(n, nq * hd)
        d = float((out[cur: cur + n] - ref).abs().max())
        assert d <= tol(dtype, max(1.0, float(ref.abs().max()))), (r, d)
        cur += n
    p = torch.softmax((qkv[0, :hd].float() * scale) @ ks[0][:lens[0], 0].float().t(), 0)
    assert float(p[77]) > 0.9


LENS8 = [2048, 2047, 1000, 700, 65, 1, 1999, 513]


def _lens64():
    g = torch.Generator().manual_seed(64)
    return [2048, 2047, 1, 64, 65] + torch.randint(1, 2049, (59,), generator=g).tolist()


@pytest.mark.parametrize("wide", [False, True, "cluster"])
@pytest.mark.parametrize("bucket", [False, True])
@pytest.mark.parametrize("hd,nq,nkv,q_len,lens,window,page", [
    (64, 32, 4, 1, [2048], None, 16),          # batch 1 at the longest context: the most key slices
    (64, 32, 4, 1, LENS8, None, 16),           # the benchmark's shape, contexts from 1 to 2,048 in one batch
    (64, 8, 1, 2, LENS8, 37, 16),              # two tokens x a group of eight = 16 rows, a window
    (128, 8, 8, 1, LENS8, None, 16),           # one query head per key/value head, head size 128
    (128, 32, 8, 1, [2048, 1000, 2047], None, 32),
    (128, 4, 1, 4, LENS8, None, 8),            # four tokens x a group of four
    (64, 4, 2, 1, _lens64(), None, 16),        # batch 64
    (128, 2, 1, 1, _lens64(), 500, 16),
], ids=["b1", "b8", "b8-q2-window", "b8-mha-hd128", "b3-hd128-page32", "b8-q4-hd128", "b64", "b64-hd128-window"])
def test_decode_attention_over_long_contexts(ops, hd, nq, nkv, q_len, lens, window, page, bucket, wide, monkeypatch):
    """Every request brings q_len tokens (q_len x group <= 16), so the decode kernels and the merge of their key
    slices run, with the slice count the engine itself picks for these sizes; `bucket` hands the kernel
    the power-of-two bucket of the longest context, as a replayed graph does, so that short requests
    have empty slices; `wide` takes the kernel with one warp per tile wherever the head size lets it (else the
    kernel that walks a slice tile by tile), "cluster" with its slices merged inside a thread-block cluster instead
    of by a kernel behind it.  Unwritten slots of the pages are NaN; one key far back carries a query."""
    from tiny_llm_b200.engine import Workspace
    monkeypatch.setattr(ops, "decode_wide_ctas", (1, 1 << 30) if wide else (1, 0))
    monkeypatch.setattr(ops, "_cluster_merge", lambda n_req, n_kv, splits: wide == "cluster" and 2 <= splits <= 8)   # at every batch
    dtype = "bfloat16"
    n_req = len(lens)
    lens = [max(l, q_len) for l in lens]
    group = nq // nkv
    assert q_len * group <= 16
    table, k_cache, v_cache, ks, vs = paged_setup(dtype, n_req, lens, nkv, hd, page, seed=hd + nq + n_req)
    g = torch.Generator().manual_seed(11)
    t = n_req * q_len
    qkv = torch.randn(t, (nq + 2 * nkv) * hd, generator=g).to(DT[dtype])
    far = 3 if lens[0] > 3 else 0
    if window is None:   # request 0's last query, first head, and its key 3 are scaled so that this score stands out
        row = q_len - 1
        qkv[row, :hd] *= 6.0
        ks[0][far, 0] = (qkv[row, :hd] / qkv[row, :hd].float().norm() * 8.0).to(DT[dtype])
        k_cache[int(table[0, far // page]), 0, far % page] = ks[0][far, 0]
    tok_req = torch.arange(n_req, dtype=torch.int32).repeat_interleave(q_len)
    pos = torch.cat([torch.arange(l - q_len, l, dtype=torch.int32) for l in lens])
    cu = torch.arange(0, t + 1, q_len, dtype=torch.int32)
    starts = torch.tensor([l - q_len for l in lens], dtype=torch.int32)
    max_kv = max(lens)
    if bucket:
        max_kv = 256
        while max_kv < max(lens):
            max_kv *= 2
        max_kv *= 2 if max_kv == max(lens) else 1     # a bucket that is strictly larger than every context
    batch = types.SimpleNamespace(token_request=tok_req.to(DEV), positions=pos.to(DEV), cu_q=cu.to(DEV),
                                  q_start=starts.to(DEV), num_requests=n_req, max_q_len=q_len, max_kv_len=max_kv)
    splits = ops._attention_splits(n_req, q_len, group, nkv, max_kv)
    assert splits > 1 or max(lens) < 128
    out = torch.full((t, nq * hd), float("nan"), dtype=DT[dtype], device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ops.paged_attention(qkv.to(DEV), nq, nkv, hd, k_cache.to(DEV), v_cache.to(DEV), table.to(DEV), batch, out,
                        scale, window, Workspace(DEV))
    out = out.float().cpu()
    assert not torch.isnan(out).any()
    for r, l in enumerate(lens):
        q = qkv[r * q_len: (r + 1) * q_len, : nq * hd].float().view(q_len, nq, hd)
        ref = pl.attention(q, ks[r].float(), vs[r].float(), pos[r * q_len: (r + 1) * q_len], window=window,
                           quant=pl.bf16_quant).reshape(q_len, nq * hd)
        d = float((out[r * q_len: (r + 1) * q_len] - ref).abs().max())
        assert d <= tol(dtype, max(1.0, float(ref.abs().max()))), (r, l, d, splits)
    if window is None:
        p = torch.softmax((qkv[q_len - 1, :hd].float() * scale) @ ks[0][:lens[0], 0].float().t(), 0)
        assert float(p[far]) > 0.9


@pytest.mark.parametrize("hd,nq,nkv", [(64, 8, 2), (128, 4, 1)])
def test_attention_beyond_the_block_table_entries_kept_in_shared_memory(ops, hd, nq, nkv):
    """Contexts of 9,000 keys in pages of 8: 1,125 block-table entries per request, more than the kernels stage in
    shared memory (512 for the mma.sync kernels, 1,024 for the tcgen05 kernel), so the later entries come
    from global memory.  A portion of 300 tokens at the end of one request (tcgen05), a decoded token of another
    (key slices), and a far key at the very beginning and one past entry 1,024."""
    from tiny_llm_b200.engine import Workspace
    dtype, page = "bfloat16", 8
    lens = [9000, 8200]
    table, k_cache, v_cache, ks, vs = paged_setup(dtype, 2, lens, nkv, hd, page, seed=hd)
    g = torch.Generator().manual_seed(31)
    scale = 1.0 / math.sqrt(hd)
    for q_lens in ([300, 0], [0, 1]):                       # the portion alone (tcgen05), then the decoded token alone
        live = [r for r in range(2) if q_lens[r]]
        t = sum(q_lens)
        qkv = torch.randn(t, (nq + 2 * nkv) * hd, generator=g).to(DT[dtype])
        r = live[0]
        for key in (2, 8600 if r == 0 else 8195):             # standout keys: block 0, and a block past the staged entries
            row = (t - 1) if key == 2 else max(0, t - 2)
            head = 0 if key == 2 else (1 if nq > 1 else 0)
            qkv[row, head * hd:(head + 1) * hd] *= 6.0
            kvh = head // (nq // nkv)
            qv = qkv[row, head * hd:(head + 1) * hd]
            ks[r][key, kvh] = (qv / qv.float().norm() * 8.0).to(DT[dtype])
            k_cache[int(table[r, key // page]), kvh, key % page] = ks[r][key, kvh]
        n = q_lens[r]
        pos = torch.arange(lens[r] - n, lens[r], dtype=torch.int32)
        batch = types.SimpleNamespace(token_request=torch.zeros(n, dtype=torch.int32, device=DEV), positions=pos.to(DEV),
                                      cu_q=torch.tensor([0, n], dtype=torch.int32, device=DEV),
                                      q_start=torch.tensor([lens[r] - n], dtype=torch.int32, device=DEV),
                                      num_requests=1, max_q_len=n, max_kv_len=lens[r])
        out = torch.full((n, nq * hd), float("nan"), dtype=DT[dtype], device=DEV)
        ops.paged_attention(qkv.to(DEV), nq, nkv, hd, k_cache.to(DEV), v_cache.to(DEV), table[r: r + 1].contiguous().to(DEV),
                            batch, out, scale, None, Workspace(DEV))
        ops.check_status()
        out = out.float().cpu()
        assert not torch.isnan(out).any()
        q = qkv[:, : nq * hd].float().view(n, nq, hd)
        ref = pl.attention(q, ks[r].float(), vs[r].float(), pos, quant=pl.bf16_quant).reshape(n, nq * hd)
        d = float((out - ref).abs().max())
        assert d <= tol(dtype, max(1.0, float(ref.abs().max()))), (q_lens, d)
        p0 = torch.softmax((qkv[n - 1, :hd].float() * scale) @ ks[r][:lens[r], 0].float().t(), 0)
        assert float(p0[2]) > 0.9                             # the far key carries its query


def test_products_at_the_sizes_of_a_2048_token_prompt(ops):
    """The persistent 128 x 256 kernel over several rounds of tiles at the TinyLlama layer sizes: gate/up
    with SiLU * up in its epilogue (2,048 x 11,264 x 2,048) and the down projection adding into the
    32-bit residual (2,048 x 2,048 x 5,632), each against a 64-bit product on the host."""
    from tiny_llm_b200.engine import Workspace
    from tiny_llm_b200.parts import interleave_gate_up
    g = torch.Generator().manual_seed(21)
    m, h, inter = 2048, 2048, 5632
    a = torch.randn(m, h, generator=g).to(torch.bfloat16)
    wg = (torch.randn(inter, h, generator=g) / math.sqrt(h)).to(torch.bfloat16)
    wu = (torch.randn(inter, h, generator=g) / math.sqrt(h)).to(torch.bfloat16)
    act = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(a.to(DEV), interleave_gate_up(wg, wu, 128).to(DEV), act, 128, Workspace(DEV))
    ops.check_status()
    ref = pl.silu(pl.linear(a.float(), wg.float())) * pl.linear(a.float(), wu.float())
    d = (act.float().cpu() - ref).abs()
    assert float(d.max()) <= tol("bfloat16", max(1.0, float(ref.abs().max()))), float(d.max())
    # down projection: adds into a residual that already holds values
    wd = (torch.randn(h, inter, generator=g) / math.sqrt(inter)).to(torch.bfloat16)
    z = pl.bf16_quant(ref).to(torch.bfloat16)
    resid0 = torch.randn(m, h, generator=g)
    resid = resid0.to(DEV)
    ops.linear(z.to(DEV), wd.to(DEV), resid, accumulate=True)
    ops.check_status()
    ref2 = (resid0.double() + pl.linear(z.double(), wd.double())).float()
    d2 = (resid.cpu() - ref2).abs()
    assert float(d2.max()) <= 5e-4 * max(1.0, float(ref2.abs().max())), float(d2.max())   # 32-bit sums of exact bfloat16 products


@pytest.mark.parametrize("m,n,k", [(512, 2048, 5632), (1024, 2048, 2048), (300, 520, 1000), (129, 256, 512), (640, 2304, 712),
                                   (200, 200, 456), (255, 96, 256), (900, 72, 96), (2048, 40, 64)])
def test_residual_adding_product_of_few_tiles_with_its_k_in_runs(ops, m, n, k):
    """Between 129 and about 1,000 tokens the residual-adding products have fewer 128 x 256 tiles than the GPU has SMs, and
    every tile's K is cut into runs that different CTAs add into the output: widths and depths that fill no tile, a
    last run that is shorter than the others, an output that already holds values; outputs narrower than a tile, whose
    sums leave in fewer staging chunks than a tile has (a chunk past the output's end must not touch a staging buffer
    that a reduction still reads)."""
    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g)).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    out0 = torch.randn(m, n, generator=g)
    out = out0.to(DEV)
    ops.linear(a.to(DEV), w.to(DEV), out, accumulate=True)
    ops.check_status()
    ref = (out0.double() + pl.linear(a.double(), w.double())).float()
    d = float((out.cpu() - ref).abs().max())
    assert d <= 5e-4 * max(1.0, float(ref.abs().max())), d   # 32-bit sums of exact bfloat16 products


@pytest.mark.parametrize("m,inter,k", [(512, 5632, 2048), (1024, 5632, 520), (600, 5632, 264), (1024, 2560, 1024), (1000, 2688, 72)])
def test_gate_up_product_with_its_last_round_in_strips(ops, m, inter, k):
    """More 128 x 256 tiles than SMs and an incomplete last round: its tiles run as four or two strips of gate columns
    with their up columns (176 tiles -> 148 + 28 x 4; 352 -> 296 + 56 x 2; 220 -> 148 + 72 x 2; 160 -> 148 + 12 x 4;
    168 -> 148 + 20 x 4 with rows that fill no tile)."""
    from tiny_llm_b200.engine import Workspace
    from tiny_llm_b200.parts import interleave_gate_up
    g = torch.Generator().manual_seed(m + inter + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    wg = (torch.randn(inter, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    wu = (torch.randn(inter, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    act = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(a.to(DEV), interleave_gate_up(wg, wu, 128).to(DEV), act, 128, Workspace(DEV))
    ops.check_status()
    ref = pl.silu(pl.linear(a.float(), wg.float())) * pl.linear(a.float(), wu.float())
    d = (act.float().cpu() - ref).abs()
    assert not torch.isnan(act).any()
    assert float(d.max()) <= tol("bfloat16", max(1.0, float(ref.abs().max()))), float(d.max())


def test_attention_refuses_sizes_it_is_not_built_for(ops):
    from tiny_llm_b200.ops import KernelError
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    batch = types.SimpleNamespace(token_request=z[:1], positions=z[:1], cu_q=z, q_start=z[:1], num_requests=1,
                                  max_q_len=1, max_kv_len=1)
    for hd in (24, 272):
        kc = torch.zeros(2, 1, 4, hd, device=DEV)
        with pytest.raises(KernelError, match="head size"):
            ops.paged_attention(torch.zeros(1, 3 * hd, device=DEV), 1, 1, hd, kc, kc.clone(),
                                torch.zeros(1, 2, dtype=torch.int32, device=DEV), batch,
                                torch.zeros(1, hd, device=DEV), 1.0)
    with pytest.raises(KernelError, match="CUDA"):
        ops.rms_norm(torch.zeros(2, 4), torch.zeros(4), 1e-5, torch.zeros(2, 4))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nq,nkv,hd,page", [(6, 3, 48, 8), (4, 1, 128, 16), (2, 2, 16, 4)])
def test_rope_kv_write(ops, dtype, nq, nkv, hd, page):
    torch.manual_seed(5)
    t, n_pages, max_pos = 23, 9, 77
    cos, sin = pl.rope_tables(max_pos, hd, 5000.0)
    qkv = torch.randn(t, (nq + 2 * nkv) * hd).to(DT[dtype])
    pos = torch.randint(0, max_pos, (t,), dtype=torch.int32)
    slots = torch.randperm(n_pages * page)[:t].to(torch.int32)
    kc = torch.zeros(n_pages, nkv, page, hd, dtype=DT[dtype], device=DEV)
    vc = torch.zeros_like(kc)
    dev = qkv.to(DEV)
    ops.rope_kv_write(dev, pos.to(DEV), cos.to(DEV), sin.to(DEV), hd, nq, nkv, hd, kc, vc, slots.to(DEV))
    q_ref = pl.apply_rope(qkv[:, : nq * hd].float().view(t, nq, hd), cos, sin, pos)
    k_ref = pl.apply_rope(qkv[:, nq * hd: (nq + nkv) * hd].float().view(t, nkv, hd), cos, sin, pos)
    v_ref = qkv[:, (nq + nkv) * hd:].view(t, nkv, hd)
    e = tol(dtype, 4.0)
    assert float((dev[:, : nq * hd].float().cpu().view(t, nq, hd) - q_ref).abs().max()) <= e
    assert torch.equal(dev[:, nq * hd:].cpu(), qkv[:, nq * hd:])           # keys and values of the row stay
    kc, vc = kc.cpu(), vc.cpu()
    for i in range(t):
        pg, off = int(slots[i]) // page, int(slots[i]) % page
        assert float((kc[pg, :, off].float() - k_ref[i]).abs().max()) <= e
        assert torch.equal(vc[pg, :, off], v_ref[i])
    written = torch.zeros(n_pages * page, dtype=torch.bool)
    written[slots.long()] = True
    assert float(kc.permute(0, 2, 1, 3).reshape(n_pages * page, -1)[~written].abs().sum()) == 0   # nothing else touched
    # a float32 accumulation buffer as the source: same queries and pages, buffer handed back zeroed
    acc = qkv.float().to(DEV)
    dev3 = torch.zeros_like(dev)
    kc3 = torch.zeros(n_pages, nkv, page, hd, dtype=DT[dtype], device=DEV)
    vc3 = torch.zeros_like(kc3)
    ops.rope_kv_write(dev3, pos.to(DEV), cos.to(DEV), sin.to(DEV), hd, nq, nkv, hd, kc3, vc3, slots.to(DEV), src=acc)
    assert torch.equal(dev3[:, : nq * hd], dev[:, : nq * hd]) and torch.equal(kc3.cpu(), kc) and torch.equal(vc3.cpu(), vc)
    assert float(acc.abs().sum()) == 0.0
    # queries only, no tables: nothing rotates, nothing is written
    q_only = torch.randn(t, nq * hd).to(DT[dtype])
    dev2 = q_only.to(DEV)
    ops.rope_kv_write(dev2, pos.to(DEV), None, None, 0, nq, nkv, hd, None, None, None)
    assert torch.equal(dev2.cpu(), q_only)


def test_argmax_takes_the_first_maximum(ops):
    torch.manual_seed(6)
    logits = torch.randn(5, 1337)
    logits[1, 700] = logits[1, 20] = 9.0
    logits[2, :] = 0.25
    logits[3, 1336] = 50.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(logits.to(DEV), out)
    assert out.cpu().tolist() == [pl.greedy(r) for r in logits] and out[1] == 20 and out[2] == 0


@pytest.mark.parametrize("vocab", [331, 32000])
def test_sample_follows_the_reference_chain(ops, vocab):
    from tiny_llm_b200.sampling import uniform_from
    torch.manual_seed(8)
    cases = [(1.0, 0, 1.0), (0.7, 50, 0.95), (0.8, 0, 0.5), (1.3, 5, 1.0), (0.5, 1, 1.0), (2.0, 40, 0.1), (0.0, 50, 0.95)]
    n = len(cases) * 6
    logits = torch.randn(n, vocab) * 3
    temps = torch.tensor([c[0] for c in cases] * 6)
    ks = torch.tensor([c[1] for c in cases] * 6, dtype=torch.int32)
    ps = torch.tensor([c[2] for c in cases] * 6)
    seeds = torch.arange(n, dtype=torch.int64) * 7919 + 3
    counters = torch.arange(n, dtype=torch.int64) % 5
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    work = torch.empty(n * vocab, device=DEV)
    ops.sample(logits.to(DEV), work, temps.to(DEV), ks.to(DEV), ps.to(DEV), seeds.to(DEV), counters.to(DEV), out)
    out = out.cpu().tolist()
    for i in range(n):
        if temps[i] <= 0:
            assert out[i] == pl.greedy(logits[i])
            continue
        ids, p = pl.sampling_distribution(logits[i], float(temps[i]), int(ks[i]), float(ps[i]))
        u = uniform_from(int(seeds[i]), int(counters[i]))
        want = pl.multinomial(ids, p, u)
        if out[i] != want:
            # only a draw within rounding of a boundary of the running sum may land on the neighbour
            cdf = torch.cumsum(p, 0)
            j = ids.tolist().index(out[i]) if out[i] in ids.tolist() else -1
            assert j >= 0, (i, "a dropped token was drawn")
            lo = float(cdf[j - 1]) if j else 0.0
            assert lo - 1e-5 <= u <= float(cdf[j]) + 1e-5, (i, out[i], want)
        assert out[i] in ids.tolist()
    # the draw depends on (seed, counter) only: the same rows in another order and batch give the same tokens
    perm = torch.randperm(n)
    out2 = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits[perm].to(DEV), work, temps[perm].to(DEV), ks[perm].to(DEV), ps[perm].to(DEV),
               seeds[perm].to(DEV), counters[perm].to(DEV), out2)
    assert out2.cpu().tolist() == [out[int(j)] for j in perm]


def test_sample_top_k_keeps_exactly_k_with_ties(ops):
    logits = torch.zeros(1, 64)
    logits[0, [5, 9, 30]] = 4.0      # three tie for two places: the lowest ids stay
    logits[0, 50] = 6.0
    draws = set()
    work = torch.empty(64, device=DEV)
    out = torch.empty(1, dtype=torch.int32, device=DEV)
    for c in range(200):
        ops.sample(logits.to(DEV), work, torch.tensor([1.0], device=DEV), torch.tensor([3], dtype=torch.int32, device=DEV),
                   torch.tensor([1.0], device=DEV), torch.tensor([11], dtype=torch.int64, device=DEV),
                   torch.tensor([c], dtype=torch.int64, device=DEV), out)
        draws.add(int(out[0]))
    assert draws == {5, 9, 50}
