"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from openvino_b200.ops import cuda as k
    k.lib()
    return k


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (16, 256, 256), (64, 4096, 4096), (100, 384, 1024), (300, 512, 448),
                                   (2048, 1024, 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_dense(ops, T, N, K, dtype):
    torch.manual_seed(0)
    x = torch.randn(T, K, device="cuda", dtype=dtype)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(dtype)
    bias = torch.randn(N, device="cuda").to(dtype)
    res = torch.randn(T, N, device="cuda").to(dtype)
    pw = ops.PackedWeight.from_dense(w, bias)
    y = ops.gemm(x, pw, residual=res)
    ops.check_status("gemm")
    ref = x.float() @ w.float().t() + bias.float() + res.float()
    assert _rel_err(y, ref) < 1e-2
    # activation epilogue, fp32 output
    y2 = ops.gemm(x, ops.PackedWeight.from_dense(w), act=ops.ACT_GELU_ERF, out_f32=True)
    ref2 = torch.nn.functional.gelu(x.float() @ w.float().t())
    assert _rel_err(y2, ref2) < 1e-2
    ops.check_status("gemm")


@pytest.mark.parametrize("T,N,K,splits", [(4, 256, 512, 1), (64, 512, 4096, 4), (64, 4096, 14336, 0), (33, 384, 1024, 8),
                                          (512, 1024, 1024, 1), (1000, 256, 2048, 1)])
def test_gemm_u4(ops, T, N, K, splits):
    from openvino_b200.utils import quant
    torch.manual_seed(1)
    gs = 128
    w = torch.randn(N, K, device="cuda") * 0.05
    q, s, z = quant.quantize_u4_asym(w, gs)
    wdq = quant.dequantize_u4(q, s, z, gs)
    pw = ops.PackedWeight.from_ir_u4(quant.pack_u4(q), s, quant.pack_u4(z), N, K, gs)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    y = ops.gemm(x, pw, splits=splits)
    ops.check_status("gemm_u4")
    ref = x.float() @ wdq.t()
    assert _rel_err(y, ref) < 1.5e-2
    # run twice: identical bits (split-K reduction order is fixed)
    y2 = ops.gemm(x, pw, splits=splits)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("fmt", ["bf16", "u4"])
@pytest.mark.parametrize("counts,block_t", [([40, 0, 300, 17], 0), ([5, 9, 1, 3, 0, 0, 7, 2], 16), ([256, 256], 128)])
def test_gemm_grouped_moe(ops, fmt, counts, block_t):
    """One launch runs every group (expert) on its own rows of stacked weights; the row offsets live on the device.
    Mode 1 (stacked along N: gate/up projections) and mode 2 (stacked along K: down projections), empty groups and
    partial row tiles included; the sorted gather / weighted combine kernels around it against plain indexing."""
    from openvino_b200.utils import quant
    torch.manual_seed(11)
    G, H, F = len(counts), 256, 384
    rows = sum(counts)
    cap = rows + 19                                      # rows past the last group hold garbage and stay untouched
    w1 = torch.randn(G, F, H, device="cuda") * 0.05      # [G, N = F, K = H]
    w2 = torch.randn(G, H, F, device="cuda") * 0.05      # [G, N = H, K = F]
    w1s = w1.reshape(G * F, H)                           # stacked along N
    w2s = w2.permute(1, 0, 2).reshape(H, G * F)          # stacked along K
    if fmt == "bf16":
        pw1 = ops.PackedWeight.from_dense(w1s.to(torch.bfloat16))
        pw2 = ops.PackedWeight.from_dense(w2s.to(torch.bfloat16))
        d1, d2 = w1s.to(torch.bfloat16).float(), w2s.to(torch.bfloat16).float()
    else:
        gs = 128
        q1, s1, z1 = quant.quantize_u4_asym(w1s, gs)
        q2, s2, z2 = quant.quantize_u4_asym(w2s, gs)
        pw1 = ops.PackedWeight.from_ir_u4(quant.pack_u4(q1), s1, quant.pack_u4(z1), G * F, H, gs)
        pw2 = ops.PackedWeight.from_ir_u4(quant.pack_u4(q2), s2, quant.pack_u4(z2), H, G * F, gs)
        d1, d2 = quant.dequantize_u4(q1, s1, z1, gs), quant.dequantize_u4(q2, s2, z2, gs)
    d1 = d1.reshape(G, F, H)
    d2 = d2.reshape(H, G, F).permute(1, 0, 2)
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    x = torch.randn(cap, H, device="cuda", dtype=torch.bfloat16)
    y1 = torch.full((cap, F), 7.0, device="cuda", dtype=torch.bfloat16)
    ops.gemm_grouped(x, pw1, offs, G, 1, out=y1, block_t=block_t)
    ops.check_status("grouped gemm, stacked along N")
    y2 = torch.full((cap, H), 7.0, device="cuda", dtype=torch.bfloat16)
    ops.gemm_grouped(y1, pw2, offs, G, 2, out=y2, block_t=block_t)
    ops.check_status("grouped gemm, stacked along K")
    o = 0
    for g, c in enumerate(counts):
        if c:
            ref1 = x[o:o + c].float() @ d1[g].t()
            assert _rel_err(y1[o:o + c], ref1) < 1.5e-2, (g, c)
            ref2 = y1[o:o + c].float() @ d2[g].t()
            assert _rel_err(y2[o:o + c], ref2) < 1.5e-2, (g, c)
        o += c
    assert torch.all(y1[rows:] == 7.0) and torch.all(y2[rows:] == 7.0)


def test_moe_sorted_gather_combine(ops):
    torch.manual_seed(12)
    T, E, k, H, e0, nloc = 300, 8, 2, 128, 2, 4
    logits = torch.randn(T, E, device="cuda")
    route = ops.moe_route_topk(logits, k)
    pos = torch.zeros(T, nloc, dtype=torch.int32, device="cuda")
    counts = torch.zeros(nloc, dtype=torch.int32, device="cuda")
    offsets = torch.zeros(nloc + 1, dtype=torch.int32, device="cuda")
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    xg = torch.zeros(T * k, H, device="cuda", dtype=torch.bfloat16)
    ops.moe_positions(route, e0, nloc, pos, counts)
    ops.moe_gather_sorted(x, pos, counts, offsets, xg)
    hit = route[:, e0:e0 + nloc] != 0
    assert counts.tolist() == hit.sum(0).tolist()
    assert offsets.tolist() == [0] + hit.sum(0).cumsum(0).tolist()
    for e in range(nloc):
        toks = hit[:, e].nonzero().flatten()
        assert torch.equal(pos[toks, e].long(), torch.arange(len(toks), device="cuda"))
        assert torch.equal(xg[offsets[e]:offsets[e + 1]], x[toks])
    assert torch.all(pos[~hit] == -1)
    # the experts' "results": row r of expert e becomes (e + 1) * row
    y = xg.clone()
    for e in range(nloc):
        y[offsets[e]:offsets[e + 1]] *= (e + 1)
    base = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    dst = base.clone()
    ops.moe_combine_sorted(y, route, pos, offsets, dst, e0, accumulate=True)
    w = (route[:, e0:e0 + nloc] * torch.arange(1, nloc + 1, device="cuda")).sum(1, keepdim=True)
    ref = base.float() + w * x.float()
    assert _rel_err(dst, ref) < 1e-2
    dst2 = torch.full_like(base, 3.0)
    ops.moe_combine_sorted(y, route, pos, offsets, dst2, e0, accumulate=False)
    assert _rel_err(dst2, w * x.float()) < 1e-2
    # silu(gate) * up over the valid rows only (the count is read on the device)
    gu = torch.randn(T * k, 2 * H, device="cuda", dtype=torch.bfloat16)
    act = torch.full((T * k, H), 5.0, device="cuda", dtype=torch.bfloat16)
    ops.silu_mul(gu, out=act, nrows=offsets[nloc:])
    n = int(offsets[nloc])
    ref = torch.nn.functional.silu(gu[:n, :H].float()) * gu[:n, H:].float()
    assert _rel_err(act[:n], ref) < 1e-2 and torch.all(act[n:] == 5.0)
    ops.check_status("moe sorted")


def test_gemm_u8(ops):
    from openvino_b200.utils import quant
    torch.manual_seed(2)
    T, N, K, gs = 48, 256, 1024, 128
    w = torch.randn(N, K, device="cuda") * 0.05
    q, s, z = quant.quantize_u8_asym(w, gs)
    wdq = ((q.float().reshape(N, K // gs, gs) - z.float().unsqueeze(-1)) * s.float().unsqueeze(-1)).reshape(N, K)
    pw = ops.PackedWeight.from_ir_u8(q, s, z, N, K, gs)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    y = ops.gemm(x, pw)
    ops.check_status("gemm_u8")
    assert _rel_err(y, x.float() @ wdq.t()) < 1.5e-2


@pytest.mark.parametrize("T,N,K", [(48, 256, 1024), (300, 384, 512), (7, 1000, 256)])
def test_gemm_f8_block_scaled(ops, T, N, K):
    """fp8 e4m3 weights with one fp32 scale per 128 x 128 tile (weight-only: activations stay bf16)."""
    from openvino_b200.utils import quant
    torch.manual_seed(4)
    w = torch.randn(N, K, device="cuda") * 0.05
    w[0, :16] = 1e-5          # lands in the fp8 sub-normal range of its tile
    q, s = quant.quantize_f8_block(w, 128)
    wdq = quant.dequantize_f8_block(q, s, 128)
    assert _rel_err(wdq, w) < 5e-2
    pw = ops.PackedWeight.from_f8_block(q, s, N, K, 128)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    y = ops.gemm(x, pw)
    ops.check_status("gemm_f8")
    assert _rel_err(y, x.float() @ wdq.t()) < 1e-2


@pytest.mark.parametrize("B,C,H,W,O,k,stride,pad,dil", [(2, 3, 32, 32, 64, 7, 2, 3, 1), (1, 64, 14, 14, 128, 3, 1, 1, 1),
                                                        (3, 32, 9, 11, 48, 3, 2, 1, 1), (2, 16, 8, 8, 32, 1, 1, 0, 1), (1, 8, 12, 12, 16, 3, 1, 2, 2)])
def test_conv2d_im2col_gemm(ops, B, C, H, W, O, k, stride, pad, dil):
    torch.manual_seed(5)
    x = torch.randn(B, C, H, W, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(O, C, k, k, device="cuda") * 0.1).to(torch.bfloat16)
    pw = ops.pack_conv_weight(w)
    y = ops.conv2d(x, pw, [k, k], [stride, stride], [pad, pad], [pad, pad], [dil, dil])
    ops.check_status("conv2d")
    ref = torch.nn.functional.conv2d(x.float(), w.float(), None, stride, pad, dil)
    assert list(y.shape) == list(ref.shape)
    assert _rel_err(y, ref) < 1e-2


@pytest.mark.parametrize("T,wmode", [(48, "bf16"), (300, "bf16"), (64, "u4"), (1000, "u4")])
def test_gemm_fused_swiglu(ops, T, wmode):
    from openvino_b200.utils import quant
    torch.manual_seed(9)
    F, K = 384, 512
    gate = torch.randn(F, K, device="cuda") * 0.05
    up = torch.randn(F, K, device="cuda") * 0.05
    w = ops.interleave_gate_up(gate, up)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    if wmode == "bf16":
        pw = ops.PackedWeight.from_dense(w.to(torch.bfloat16))
        gq, uq = gate.to(torch.bfloat16).float(), up.to(torch.bfloat16).float()
    else:
        q, s, z = quant.quantize_u4_asym(w, 128)
        pw = ops.PackedWeight.from_ir_u4(quant.pack_u4(q), s, quant.pack_u4(z), 2 * F, K, 128)
        wd = quant.dequantize_u4(q, s, z, 128).float().reshape(F // 64, 2, 64, K)
        gq, uq = wd[:, 0].reshape(F, K), wd[:, 1].reshape(F, K)
    y = ops.gemm(x, pw, act=ops.ACT_SWIGLU)
    ops.check_status("gemm swiglu")
    assert list(y.shape) == [T, F]
    ref = torch.nn.functional.silu(x.float() @ gq.t()) * (x.float() @ uq.t())
    assert _rel_err(y, ref) < 2e-2


def test_gumbel_sampling_matches_softmax_and_shards_agree(ops):
    torch.manual_seed(8)
    V = 512
    logits = (torch.randn(1, V, device="cuda") * 2.0).to(torch.bfloat16)
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    rows = logits.expand(4096, V).contiguous()
    counts = torch.zeros(V, device="cuda")
    for it in range(8):
        step.fill_(it)
        ids = ops.sample_gumbel(rows, 0.8, seed=11, step=step)
        counts += torch.bincount(ids.long(), minlength=V).float()
    ops.check_status("sample_gumbel")
    p = torch.softmax(logits.float()[0] / 0.8, -1)
    freq = counts / counts.sum()
    top = torch.topk(p, 20).indices
    assert (freq[top] - p[top]).abs().max() < 0.01 and (freq - p).abs().sum() < 0.12
    # two vocabulary shards with global indices give the full-vocabulary draw
    x = (torch.randn(32, V, device="cuda") * 3.0).to(torch.bfloat16)
    full_max = torch.empty(32, device="cuda")
    full = ops.sample_gumbel(x, 1.3, seed=5, step=step, out_max=full_max)
    m0, m1 = torch.empty(32, device="cuda"), torch.empty(32, device="cuda")
    i0 = ops.sample_gumbel(x[:, :256].contiguous(), 1.3, seed=5, step=step, vocab_offset=0, out_max=m0)
    i1 = ops.sample_gumbel(x[:, 256:].contiguous(), 1.3, seed=5, step=step, vocab_offset=256, out_max=m1)
    merged = torch.where(m0 >= m1, i0, i1 + 256)
    assert torch.equal(merged, full) and torch.equal(torch.maximum(m0, m1), full_max)


def test_gumbel_noise_stays_finite_on_a_large_flat_vocabulary(ops):
    # 64 rows x 128256 tokens x 4 steps = 33M uniforms: with a 24-bit mapping about two of them would round to exactly 1
    V = 128256
    logits = torch.zeros(64, V, device="cuda", dtype=torch.bfloat16)
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    out_max = torch.empty(64, device="cuda")
    for it in range(4):
        step.fill_(it)
        ids = ops.sample_gumbel(logits, 1.0, seed=3, step=step, out_max=out_max)
        assert torch.isfinite(out_max).all() and int(ids.min()) >= 0 and int(ids.max()) < V
    ops.check_status("sample_gumbel")


def test_act_quant_fp8_groups_of_128(ops):
    torch.manual_seed(6)
    x = (torch.randn(37, 512, device="cuda") * torch.logspace(-2, 1, 512, device="cuda")).to(torch.bfloat16)
    q, s = ops.act_quant_fp8(x)
    ops.check_status("act_quant_fp8")
    xf = x.float().reshape(37, 4, 128)
    want_s = xf.abs().amax(-1) / 448.0
    assert torch.allclose(s, want_s, rtol=1e-5), (s - want_s).abs().max()
    deq = q.view(torch.float8_e4m3fn).float().reshape(37, 4, 128) * s.unsqueeze(-1)
    assert _rel_err(deq, xf) < 4e-2                       # e4m3: 3 mantissa bits
    ref_q = (xf / want_s.unsqueeze(-1)).to(torch.float8_e4m3fn).view(torch.uint8).reshape(37, 512)
    assert (q == ref_q).float().mean() > 0.98          # x * (1 / scale) against x / scale: the last bit may differ on ties


def test_kv_block_copy_and_lora(ops):
    torch.manual_seed(7)
    k = torch.randn(12, 8, 16, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(12, 8, 16, 128, device="cuda", dtype=torch.bfloat16)
    k0, v0 = k.clone(), v.clone()
    src = torch.tensor([1, 5, 7], dtype=torch.int32, device="cuda")
    dst = torch.tensor([2, 9, 7], dtype=torch.int32, device="cuda")
    ops.kv_block_copy(k, v, src, dst)
    ops.check_status("kv_block_copy")
    want_k, want_v = k0.clone(), v0.clone()
    want_k[dst.long()], want_v[dst.long()] = k0[src.long()], v0[src.long()]
    assert torch.equal(k, want_k) and torch.equal(v, want_v)
    x = torch.randn(40, 256, device="cuda", dtype=torch.bfloat16)
    a = (torch.randn(64, 256, device="cuda") * 0.05).to(torch.bfloat16)
    b = (torch.randn(384, 64, device="cuda") * 0.05).to(torch.bfloat16)
    y = torch.randn(40, 384, device="cuda", dtype=torch.bfloat16)
    out = ops.lora_apply(x, ops.PackedWeight.from_dense(a), ops.PackedWeight.from_dense(b), y, alpha=0.5)
    ref = y.float() + 0.5 * (x.float() @ a.float().t()) @ b.float().t()
    assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("rows,cols", [(3, 128), (64, 4096), (17, 8192), (5, 14336)])
def test_rmsnorm(ops, rows, cols):
    torch.manual_seed(3)
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    r = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(cols, device="cuda", dtype=torch.bfloat16)
    y = ops.rmsnorm(x, g, 1e-5)
    xf = x.float()
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()
    assert _rel_err(y, ref) < 5e-3
    ro = torch.empty_like(x)
    y2 = ops.rmsnorm(x, g, 1e-5, residual=r, residual_out=ro)
    h = (x.float() + r.float()).to(torch.bfloat16).float()
    ref2 = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()
    assert _rel_err(y2, ref2) < 5e-3
    assert _rel_err(ro, h) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_layernorm(ops, dtype):
    torch.manual_seed(4)
    x = torch.randn(33, 1024, device="cuda", dtype=dtype)
    r = torch.randn(33, 1024, device="cuda", dtype=dtype)
    g = torch.randn(1024, device="cuda", dtype=dtype)
    b = torch.randn(1024, device="cuda", dtype=dtype)
    y = ops.layernorm(x, g, b, 1e-12, residual=r)
    ref = torch.nn.functional.layer_norm(x.float() + r.float(), (1024,), g.float(), b.float(), 1e-12)
    assert _rel_err(y, ref) < 5e-3


def test_silu_mul_embedding_argmax_add(ops):
    torch.manual_seed(5)
    gu = torch.randn(37, 2 * 1024, device="cuda", dtype=torch.bfloat16)
    y = ops.silu_mul(gu)
    ref = torch.nn.functional.silu(gu[:, :1024].float()) * gu[:, 1024:].float()
    assert _rel_err(y, ref) < 5e-3
    table = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (77,), device="cuda")
    assert torch.equal(ops.embedding(ids, table), table[ids])
    logits = torch.randn(9, 128256, device="cuda", dtype=torch.bfloat16)
    am = ops.argmax(logits)
    ref_max = logits.float().max(dim=-1).values
    assert torch.equal(logits.float().gather(1, am[:, None])[:, 0], ref_max)
    # first index on ties
    logits[:, 5] = 100.0
    logits[:, 77] = 100.0
    assert torch.equal(ops.argmax(logits), torch.full((9,), 5, device="cuda"))
    a = torch.randn(64, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(64, 512, device="cuda", dtype=torch.bfloat16)
    assert _rel_err(ops.add(a, b), a.float() + b.float()) < 5e-3


def _rope_ref(x, pos, theta):
    # x [T, H, D] float; half-rotate (LLaMA) convention
    T, H, D = x.shape
    inv = theta ** (-torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D)
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def _make_paged_batch(q_lens, past_lens, block_size, device, shuffle=True):
    """Block tables for a ragged batch; returns descriptors and total block count."""
    B = len(q_lens)
    nblocks = [(p + q + block_size - 1) // block_size for p, q in zip(past_lens, q_lens)]
    total = sum(nblocks)
    perm = torch.randperm(total) if shuffle else torch.arange(total)
    block_indices = perm.to(torch.int32)
    bib = [0]
    for n in nblocks:
        bib.append(bib[-1] + n)
    sb = [0]
    for q in q_lens:
        sb.append(sb[-1] + q)
    to = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return to(past_lens), to(sb), block_indices.to(device), to(bib), total


def _attn_ref(q, k_all, v_all, q_lens, past_lens, Hq, Hkv, D, scale, window=0):
    """q [T, Hq, D] fp32; k_all/v_all: list per sequence of [ctx, Hkv, D] fp32."""
    outs = []
    t = 0
    G = Hq // Hkv
    for b, (ql, pl) in enumerate(zip(q_lens, past_lens)):
        qb = q[t:t + ql]                                  # [ql, Hq, D]
        kb = k_all[b].repeat_interleave(G, dim=1)         # [ctx, Hq, D]
        vb = v_all[b].repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->hqk", qb, kb) * scale
        ctx = pl + ql
        qpos = pl + torch.arange(ql, device=q.device)
        kpos = torch.arange(ctx, device=q.device)
        mask = kpos[None, :] <= qpos[:, None]
        if window > 0:
            mask &= kpos[None, :] > (qpos[:, None] - window)
        s = s.masked_fill(~mask[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        outs.append(torch.einsum("hqk,khd->qhd", p, vb))
        t += ql
    return torch.cat(outs, dim=0)


@pytest.mark.parametrize("q_lens,past_lens,Hq,Hkv", [
    ([5], [0], 4, 1),
    ([40, 17, 128], [0, 3, 70], 8, 2),
    ([1, 1, 1, 1], [0, 15, 16, 300], 8, 2),            # decode
    ([1] * 7, [5, 1000, 77, 256, 31, 32, 511], 32, 8),  # decode, GQA 4
    ([200, 1], [56, 9], 32, 8),                         # mixed
    ([700, 130, 33], [330, 900, 0], 32, 8),             # long contexts: many key tiles per query tile, both stages reused
    ([300, 520], [0, 64], 8, 8),                        # one query head per KV head
    ([260], [100], 16, 2),                              # eight query heads per KV head
])
def test_rope_kv_write_and_paged_attention(ops, q_lens, past_lens, Hq, Hkv):
    torch.manual_seed(6)
    D, bs, theta = 128, 16, 500000.0
    dev = "cuda"
    pl_t, sb_t, bi_t, bib_t, total_blocks = _make_paged_batch(q_lens, past_lens, bs, dev)
    T = sum(q_lens)
    k_cache = torch.zeros(total_blocks, Hkv, bs, D, device=dev, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    # history: fill the cache with past tokens through the same write kernel
    k_hist, v_hist = [], []
    for b, pl in enumerate(past_lens):
        kh = torch.randn(pl, Hkv, D, device=dev).to(torch.bfloat16)
        vh = torch.randn(pl, Hkv, D, device=dev).to(torch.bfloat16)
        k_hist.append(kh)
        v_hist.append(vh)
        blocks = bi_t[bib_t[b]:bib_t[b + 1]].long()
        for j in range(pl):
            k_cache[blocks[j // bs], :, j % bs] = kh[j]
            v_cache[blocks[j // bs], :, j % bs] = vh[j]
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev).to(torch.bfloat16)
    positions, slots = [], []
    for b, (ql, pl) in enumerate(zip(q_lens, past_lens)):
        blocks = bi_t[bib_t[b]:bib_t[b + 1]].long().tolist()
        for j in range(pl, pl + ql):
            positions.append(j)
            slots.append(blocks[j // bs] * bs + j % bs)
    positions = torch.tensor(positions, dtype=torch.int32, device=dev)
    slots = torch.tensor(slots, dtype=torch.int32, device=dev)
    qkv0 = qkv.clone()
    ops.rope_kv_write(qkv, positions, slots, k_cache, v_cache, Hq, Hkv, D, theta, bs)
    q_ref = _rope_ref(qkv0[:, : Hq * D].float().reshape(T, Hq, D), positions, theta)
    k_new = _rope_ref(qkv0[:, Hq * D:(Hq + Hkv) * D].float().reshape(T, Hkv, D), positions, theta)
    v_new = qkv0[:, (Hq + Hkv) * D:].float().reshape(T, Hkv, D)
    assert _rel_err(qkv[:, : Hq * D].reshape(T, Hq, D), q_ref) < 5e-3
    # gather cache rows of the new tokens
    kc = k_cache.permute(0, 2, 1, 3).reshape(-1, Hkv, D)[slots.long()]
    vc = v_cache.permute(0, 2, 1, 3).reshape(-1, Hkv, D)[slots.long()]
    assert _rel_err(kc, k_new) < 5e-3
    assert torch.equal(vc.float(), v_new)

    scale = 1.0 / math.sqrt(D)
    out = ops.paged_attention(qkv, k_cache, v_cache, pl_t, sb_t, bi_t, bib_t, Hq, Hkv, D, scale=scale,
                              max_context_len=max(p + q for p, q in zip(past_lens, q_lens)), max_q_len=max(q_lens))
    ops.check_status("paged_attention")
    k_all, v_all = [], []
    t = 0
    for b, ql in enumerate(q_lens):
        k_all.append(torch.cat([k_hist[b].float(), kc[t:t + ql].float()], dim=0))
        v_all.append(torch.cat([v_hist[b].float(), vc[t:t + ql].float()], dim=0))
        t += ql
    ref = _attn_ref(qkv[:, : Hq * D].float().reshape(T, Hq, D), k_all, v_all, q_lens, past_lens, Hq, Hkv, D, scale)
    assert _rel_err(out.reshape(T, Hq, D), ref) < 1e-2


@pytest.mark.parametrize("q_lens,past_lens,Hq,Hkv", [
    ([1, 1, 1, 1], [0, 15, 16, 300], 8, 2),             # decode
    ([1] * 5, [5, 1000, 77, 256, 511], 32, 8),          # decode, split over the keys
    ([40, 17, 128], [0, 3, 70], 8, 2),                  # prefill with history
    ([200, 1], [56, 9], 32, 8),                         # mixed
    ([90], [300], 4, 4),
])
def test_u8_kv_cache_write_and_attention(ops, q_lens, past_lens, Hq, Hkv):
    """KV_CACHE_PRECISION = u8: rows are quantised per (token, head) by the write kernel; decode and prefill attention read
    the bytes. Reference: fp32 attention over the dequantised cache ((byte - zero point) * scale)."""
    torch.manual_seed(16)
    D, bs, theta, dev = 128, 16, 10000.0, "cuda"
    pl_t, sb_t, bi_t, bib_t, total_blocks = _make_paged_batch(q_lens, past_lens, bs, dev)
    B = len(q_lens)
    k_cache = torch.zeros(total_blocks, Hkv, bs, D, device=dev, dtype=torch.uint8)
    v_cache = torch.zeros_like(k_cache)
    k_meta = torch.zeros(total_blocks, Hkv, bs, 2, device=dev, dtype=torch.float16)
    v_meta = torch.zeros_like(k_meta)

    def write(n_tok_per_seq, start_per_seq):
        """Runs the write kernel for tokens [start, start + n) of every sequence; returns (qkv after RoPE, raw qkv, positions)."""
        pos, slots = [], []
        for b in range(B):
            blocks = bi_t[bib_t[b]:bib_t[b + 1]].long().tolist()
            for j in range(start_per_seq[b], start_per_seq[b] + n_tok_per_seq[b]):
                pos.append(j)
                slots.append(blocks[j // bs] * bs + j % bs)
        T = len(pos)
        if T == 0:
            return None, None, None, None
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev).to(torch.bfloat16)
        raw = qkv.clone()
        pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)
        slots_t = torch.tensor(slots, dtype=torch.int32, device=dev)
        ops.rope_kv_write_u8(qkv, pos_t, slots_t, k_cache, v_cache, k_meta, v_meta, Hq, Hkv, D, theta, bs)
        return qkv, raw, pos_t, slots_t

    write(past_lens, [0] * B)                                        # history
    qkv, raw, pos_t, slots_t = write(q_lens, past_lens)              # the step's tokens
    T = sum(q_lens)
    # the write: queries rotated in place, rows quantised within half a step of the fp32 value
    q_ref = _rope_ref(raw[:, : Hq * D].float().reshape(T, Hq, D), pos_t, theta)
    assert _rel_err(qkv[:, : Hq * D].reshape(T, Hq, D), q_ref) < 5e-3
    k_new = _rope_ref(raw[:, Hq * D:(Hq + Hkv) * D].float().reshape(T, Hkv, D), pos_t, theta)
    v_new = raw[:, (Hq + Hkv) * D:].float().reshape(T, Hkv, D)

    def deq(cache, meta):
        return (cache.float() - meta[..., 1:2].float()) * meta[..., 0:1].float()
    kd, vd = deq(k_cache, k_meta), deq(v_cache, v_meta)
    kc = kd.permute(0, 2, 1, 3).reshape(-1, Hkv, D)[slots_t.long()]
    vc = vd.permute(0, 2, 1, 3).reshape(-1, Hkv, D)[slots_t.long()]
    for got, want in ((kc, k_new), (vc, v_new)):
        step = (want.amax(-1) - want.amin(-1)) / 255.0
        assert ((got - want).abs() <= 0.75 * step.unsqueeze(-1) + 1e-3).all()

    out = ops.paged_attention(qkv, k_cache, v_cache, pl_t, sb_t, bi_t, bib_t, Hq, Hkv, D, scale=1.0 / math.sqrt(D),
                              max_context_len=max(p + q for p, q in zip(past_lens, q_lens)), max_q_len=max(q_lens), k_meta=k_meta, v_meta=v_meta)
    ops.check_status("paged_attention u8")
    k_all, v_all = [], []
    for b in range(B):
        blocks = bi_t[bib_t[b]:bib_t[b + 1]].long()
        ctx = past_lens[b] + q_lens[b]
        k_all.append(kd[blocks].permute(0, 2, 1, 3).reshape(-1, Hkv, D)[:ctx])
        v_all.append(vd[blocks].permute(0, 2, 1, 3).reshape(-1, Hkv, D)[:ctx])
    ref = _attn_ref(qkv[:, : Hq * D].float().reshape(T, Hq, D), k_all, v_all, q_lens, past_lens, Hq, Hkv, D, 1 / math.sqrt(D))
    assert _rel_err(out.reshape(T, Hq, D), ref) < 1e-2


def test_paged_attention_sliding_window(ops):
    torch.manual_seed(7)
    Hq, Hkv, D, bs = 8, 2, 128, 16
    for q_lens, past_lens in ([[90], [40]], [[1, 1], [200, 37]]):
        pl_t, sb_t, bi_t, bib_t, total_blocks = _make_paged_batch(q_lens, past_lens, bs, "cuda")
        T = sum(q_lens)
        k_cache = torch.randn(total_blocks, Hkv, bs, D, device="cuda").to(torch.bfloat16)
        v_cache = torch.randn(total_blocks, Hkv, bs, D, device="cuda").to(torch.bfloat16)
        q = torch.randn(T, Hq * D, device="cuda").to(torch.bfloat16)
        out = ops.paged_attention(q, k_cache, v_cache, pl_t, sb_t, bi_t, bib_t, Hq, Hkv, D,
                                  max_context_len=max(p + q_ for p, q_ in zip(past_lens, q_lens)),
                                  max_q_len=max(q_lens), sliding_window=32)
        k_all, v_all = [], []
        for b in range(len(q_lens)):
            blocks = bi_t[bib_t[b]:bib_t[b + 1]].long()
            ctx = past_lens[b] + q_lens[b]
            k_all.append(k_cache[blocks].permute(0, 2, 1, 3).reshape(-1, Hkv, D)[:ctx].float())
            v_all.append(v_cache[blocks].permute(0, 2, 1, 3).reshape(-1, Hkv, D)[:ctx].float())
        ref = _attn_ref(q.float().reshape(T, Hq, D), k_all, v_all, q_lens, past_lens, Hq, Hkv, D, 1 / math.sqrt(D), 32)
        assert _rel_err(out.reshape(T, Hq, D), ref) < 1e-2


@pytest.mark.parametrize("S", [200, 384, 1000])
@pytest.mark.parametrize("dtype,D", [(torch.float16, 64), (torch.bfloat16, 128), (torch.bfloat16, 64), (torch.float16, 128)])
def test_sdpa_dense(ops, dtype, D, S):
    torch.manual_seed(8)
    B, H = 3, 4
    qkv = torch.randn(B * S, 3 * H * D, device="cuda").to(dtype)
    q, k, v = qkv[:, : H * D], qkv[:, H * D: 2 * H * D], qkv[:, 2 * H * D:]
    out = ops.sdpa_dense(q, k, v, B, S, H, D, ld=3 * H * D)
    qf, kf, vf = [t.float().reshape(B, S, H, D).transpose(1, 2) for t in (q, k, v)]
    ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf).transpose(1, 2).reshape(B * S, H * D)
    assert _rel_err(out, ref) < 1e-2


def test_sampling_kernel(ops):
    torch.manual_seed(11)
    V = 1000
    logits = (torch.randn(6, V, device="cuda") * 2).to(torch.bfloat16)
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    greedy = logits.float().argmax(-1).int()
    # top_k = 1 and a tiny nucleus both reduce to the argmax
    assert torch.equal(ops.sample(logits, 1.0, top_k=1, seed=3, step=step), greedy)
    assert torch.equal(ops.sample(logits, 1.0, top_p=1e-4, seed=4, step=step), greedy)
    assert torch.equal(ops.sample(logits, 0.01, seed=5, step=step), greedy)
    # the same (seed, step) repeats, another step differs somewhere
    a = ops.sample(logits, 1.0, seed=7, step=step)
    b = ops.sample(logits, 1.0, seed=7, step=step)
    assert torch.equal(a, b)
    draws = []
    for _ in range(40):
        ops.bump(step)
        draws.append(ops.sample(logits, 1.0, top_k=5, seed=7, step=step))
    draws = torch.stack(draws)
    fifth = logits.float().topk(5, -1).values[:, -1]           # ties with the 5th value stay in the kept set
    picked = torch.gather(logits.float(), 1, draws.t().long())  # [rows, draws]
    assert (picked >= fifth[:, None]).all()
    assert len({tuple(d.tolist()) for d in draws}) > 5
    # frequencies follow the softmax: small vocabulary, many draws
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0, -30.0, 0.5, 0.5, 1.5]], device="cuda").to(torch.bfloat16).repeat(512, 1)
    counts = torch.zeros(8)
    for _ in range(8):
        ops.bump(step)
        counts += torch.bincount(ops.sample(small, 1.0, seed=9, step=step).cpu().long(), minlength=8).float()
    want = torch.softmax(small[0].float().cpu(), -1)
    assert (counts / counts.sum() - want).abs().max() < 0.03
    # nucleus: with top_p = 0.5 only the most likely tokens whose mass reaches 0.5 can appear
    ops.bump(step)
    nuc = ops.sample(small, 1.0, top_p=0.5, seed=10, step=step).cpu()
    order = want.argsort(descending=True)
    keep = order[: int((want[order].cumsum(0) < 0.5).sum()) + 1].tolist()
    assert set(nuc.tolist()) <= set(keep)


def test_bounded_wait_reports_a_timeout_and_the_context_survives(ops):
    """Failure detection on the device: a wait on a flag that nobody sets runs out of polls, the status word says so,
    and the next kernels run normally."""
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    ops.wait_flag(flag, 1, max_polls=20000, result=res)          # a few milliseconds
    assert ops.read_status() == 2 and int(res.item()) == 0        # STATUS_PEER_TIMEOUT
    assert ops.read_status() == 0                                 # reading clears the word
    flag.fill_(3)
    ops.wait_flag(flag, 3, max_polls=20000, result=res)
    assert ops.read_status() == 0 and int(res.item()) == 1
    x = torch.randn(4, 256, device="cuda", dtype=torch.bfloat16)
    y = ops.rmsnorm(x, torch.ones(256, device="cuda", dtype=torch.bfloat16), 1e-5)
    assert torch.isfinite(y.float()).all()
