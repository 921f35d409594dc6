"""Block-scaled MXFP8 kernels against the fp32 emulation in `ops.reference` (quantise -> expand -> fp32 matmul).

The quantiser must agree bit for bit with the emulation (same power-of-two scale rule, round-to-nearest-even e4m3), so the
GEMM is compared against the product of the expanded operands with only the bf16 output rounding as tolerance.
"""
import pytest
import torch

from gpt_moe_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(scope="module")
def ops():
    from gpt_moe_b200.ops import cuda_ops
    cuda_ops.ext().reset_status()
    yield cuda_ops
    cuda_ops.check_status()


def unpack_scales(sf: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """[records * 512] bytes -> fp32 scales [rows, k / 32] following the record layout of the kernels."""
    kb = (k + 127) // 128
    r = torch.arange(rows, device=sf.device)[:, None]
    g = torch.arange(k // 32, device=sf.device)[None, :]
    off = ((r // 128) * kb + g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4
    e = sf.view(-1)[off].to(torch.int32)
    return (e << 23).view(torch.float32)


@pytest.mark.parametrize("rows,cols", [(256, 128), (1000, 768), (130, 3072)])
def test_quantize_matches_emulation(ops, rows, cols):
    torch.manual_seed(0)
    x = (torch.randn(rows, cols, device="cuda") * torch.logspace(-6, 4, cols, device="cuda")).bfloat16()
    x[3, :64] = 0
    q, sf = ops.ext().mxfp8_quantize(x)
    want_q, want_s = ref.mxfp8_quantize(x.float(), -1)
    assert torch.equal(unpack_scales(sf[0], rows, cols), want_s)
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), want_q.float())
    # both weight layouts from one pass: row-wise (blocks along the columns) and transposed (blocks along the original rows)
    if rows % 32 == 0:
        q2, sf2, qt, sft = ops.ext().mxfp8_quantize_weight(x)
        assert torch.equal(q2, q) and torch.equal(unpack_scales(sf2[0], rows, cols), want_s)
        want_q, want_s = ref.mxfp8_quantize(x.float().t().contiguous(), -1)
        assert torch.equal(unpack_scales(sft[0], cols, rows), want_s)
        assert torch.equal(qt.view(torch.float8_e4m3fn).float(), want_q.float())


def test_quantize_weight_batched(ops):
    torch.manual_seed(5)
    w = (torch.randn(3, 256, 384, device="cuda") * 0.05).bfloat16()
    q, sf, qt, sft = ops.ext().mxfp8_quantize_weight(w)
    for z in range(3):
        want_q, want_s = ref.mxfp8_quantize(w[z].float(), -1)
        assert torch.equal(q[z].view(torch.float8_e4m3fn).float(), want_q.float())
        assert torch.equal(unpack_scales(sf[z], 256, 384), want_s)
        want_q, want_s = ref.mxfp8_quantize(w[z].float().t().contiguous(), -1)
        assert torch.equal(qt[z].view(torch.float8_e4m3fn).float(), want_q.float())
        assert torch.equal(unpack_scales(sft[z], 384, 256), want_s)


def _check_copy(q, sf, bf16_rows, rows):
    """The emitted copy equals the reference quantisation of the bf16 tensor the kernel wrote, bit for bit."""
    cols = bf16_rows.shape[1]
    want_q, want_s = ref.mxfp8_quantize(bf16_rows[:rows].float(), -1)
    assert torch.equal(unpack_scales(sf, rows, cols), want_s)
    assert torch.equal(q[:rows].view(torch.float8_e4m3fn).float(), want_q.float())


def test_producers_emit_the_quantised_copy_of_what_they_write(ops):
    """RMSNorm (+ residual), expert gather, activation forward / backward, combine backward and the RoPE / QK-norm backward
    write e4m3 payload + scale records of exactly their bf16 output (oracle: `ops.reference.mxfp8_quantize`)."""
    c = ops.ext()
    torch.manual_seed(6)
    tokens, d, experts, top_k, h = 777, 256, 4, 2, 384
    # RMSNorm with the residual update
    x = torch.randn(tokens, d, device="cuda")
    branch = torch.randn(tokens, d, device="cuda").bfloat16()
    w = torch.rand(d, device="cuda") + 0.5
    beta = torch.tensor([0.7], device="cuda")
    y, _, _, yq, ysf = c.rmsnorm_fwd(x, w, 1e-6, branch, None, beta, True)
    y_plain = c.rmsnorm_fwd(x, w, 1e-6, branch, None, beta)[0]
    assert torch.equal(y, y_plain)
    _check_copy(yq, ysf, y, tokens)
    # routing + gather
    idx = torch.randint(0, experts, (tokens, top_k), device="cuda")
    idx[:, 0] = torch.where(idx[:, 0] == 2, torch.zeros_like(idx[:, 0]), idx[:, 0])          # expert 2 mostly empty
    dest, src, seg, counts, tiles, meta = c.route(idx, experts)
    hidden = torch.randn(tokens, d, device="cuda").bfloat16()
    packed, pq, psf = c.gather_rows(hidden, src, meta, top_k, True)
    used = int(meta[1].item())
    assert torch.equal(packed[:used], c.gather_rows(hidden, src, meta, top_k)[0][:used])
    _check_copy(pq, psf, packed, used)
    # activations on the padded rows (SwiGLU and relu^2)
    for name, in_w in (("swiglu", 2 * h), ("relu2", h)):
        pre = torch.randn(packed.shape[0], in_w, device="cuda").bfloat16()
        act, aq, asf = c.activation_fwd(pre, name, meta, True)
        assert torch.equal(act[:used], c.activation_fwd(pre, name, meta)[0][:used])
        _check_copy(aq, asf, act, used)
        dact = torch.randn(packed.shape[0], h, device="cuda").bfloat16()
        dpre, dq, dsf = c.activation_bwd(dact, pre, name, meta, True)
        assert torch.equal(dpre[:used], c.activation_bwd(dact, pre, name, meta)[0][:used])
        _check_copy(dq, dsf, dpre, used)
    # combine backward
    gates = torch.rand(tokens, top_k, device="cuda")
    yrows = torch.randn(packed.shape[0], d, device="cuda").bfloat16()
    dout = torch.randn(tokens, d, device="cuda").bfloat16()
    dy, dg, gq, gsf = c.combine_bwd(dout, yrows, src, gates, meta, True)
    dy2, dg2 = c.combine_bwd(dout, yrows, src, gates, meta)
    assert torch.equal(dy[:used], dy2[:used]) and torch.equal(dg, dg2)
    _check_copy(gq, gsf, dy, used)
    # RoPE / QK-norm backward on packed [q | k | v] gradient rows, in place
    t, hq, hk, hd = 512, 4, 2, 64
    width = (hq + 2 * hk) * hd
    qkv = torch.randn(t, width, device="cuda").bfloat16()
    pos = torch.arange(256, device="cuda").float()[:, None] * (10000.0 ** (-torch.arange(hd // 2, device="cuda").float() / (hd // 2)))[None, :]
    cos, sin = pos.cos().contiguous(), pos.sin().contiguous()
    qs, ks = torch.rand(hq, device="cuda") + 0.5, torch.rand(hk, device="cuda") + 0.5
    g = torch.randn(t, width, device="cuda").bfloat16()
    g_ref = g.clone()
    (ds_ref,) = c.rope_qknorm_bwd(qkv, g_ref, g_ref, cos, sin, qs, ks, 256, hq, hk, hd, 1e-6, True, -3e38, 5.0)
    ds, gq, gsf = c.rope_qknorm_bwd(qkv, g, g, cos, sin, qs, ks, 256, hq, hk, hd, 1e-6, True, -3e38, 5.0, None, True)
    assert torch.equal(g, g_ref) and torch.equal(ds, ds_ref)
    _check_copy(gq, gsf, g, t)
    # attention forward: the epilogue writes the copy of the token-major output rows (operand of the output projection)
    b_, t_, h_ = 2, 256, 4
    packed_qkv = torch.randn(b_, t_, 3 * h_ * 64, device="cuda").bfloat16()
    qh = packed_qkv[..., : h_ * 64].unflatten(-1, (h_, 64))
    kh = packed_qkv[..., h_ * 64: 2 * h_ * 64].unflatten(-1, (h_, 64))
    vh = packed_qkv[..., 2 * h_ * 64:].unflatten(-1, (h_, 64))
    out, lse, oq, osf = c.attn_fwd(qh, kh, vh, 100, 0.125, 0.0, None, True)
    out_plain, _ = c.attn_fwd(qh, kh, vh, 100, 0.125)
    assert torch.equal(out, out_plain)
    _check_copy(oq, osf, out.reshape(b_ * t_, h_ * 64), b_ * t_)
    # the same through the kernel with one query tile per CTA (sequence lengths that are not a multiple of 256, document masks)
    out1, _, oq1, osf1 = c.attn_fwd(qh, kh, vh, 100, 0.125, 0.0, None, True, True)
    _check_copy(oq1, osf1, out1.reshape(b_ * t_, h_ * 64), b_ * t_)


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (1000, 768, 768), (4096, 2304, 768), (200, 1000, 256)])
def test_gemm_mxfp8_dense(ops, m, n, k):
    torch.manual_seed(1)
    c = ops.ext()
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    aq, asf = c.mxfp8_quantize(a)
    bq, bsf = c.mxfp8_quantize(b)
    d = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    c.gemm_mxfp8(aq, asf, bq, bsf, d)
    want = ref.mxfp8_linear(a.float(), b.float())
    assert rel(d, want) < 4e-3
    assert rel(d, a.float() @ b.float().t()) < 6e-2          # and the quantisation error itself is the expected few percent


def test_gemm_mxfp8_batched_and_grouped(ops):
    torch.manual_seed(2)
    c = ops.ext()
    a = torch.randn(3, 256, 256, device="cuda").bfloat16()
    b = torch.randn(3, 384, 256, device="cuda").bfloat16()
    aq, asf = c.mxfp8_quantize(a)
    bq, bsf = c.mxfp8_quantize(b)
    d = torch.empty(3, 256, 384, device="cuda", dtype=torch.bfloat16)
    c.gemm_mxfp8(aq, asf, bq, bsf, d, 0.5)
    want = torch.stack([0.5 * ref.mxfp8_linear(a[i].float(), b[i].float()) for i in range(3)])
    assert rel(d, want) < 4e-3
    counts, e, n, k = [0, 256, 512, 256], 4, 640, 256                     # expert segments are padded to the 256 rows of a CTA pair
    rows = sum(counts)
    x = torch.randn(rows + 256, k, device="cuda").bfloat16()          # one spare pair tile beyond the routed rows
    w = torch.randn(e, n, k, device="cuda").bfloat16()
    tiles = torch.tensor(sum([[i] * (cnt // 128) for i, cnt in enumerate(counts)], []) + [0, 0], dtype=torch.int32, device="cuda")
    meta = torch.tensor([rows // 128, rows], dtype=torch.int32, device="cuda")
    xq, xsf = c.mxfp8_quantize(x, meta[1:2])
    wq, wsf = c.mxfp8_quantize(w)
    y = torch.zeros(rows + 256, n, device="cuda", dtype=torch.bfloat16)
    c.gemm_mxfp8(xq, xsf, wq, wsf, y, 1.0, tiles, meta)
    starts = [0, 0, 256, 768]
    want = torch.cat([ref.mxfp8_linear(x[s:s + cnt].float(), w[i].float()) for i, (s, cnt) in enumerate(zip(starts, counts))])
    assert rel(y[:rows], want) < 4e-3
    assert y[rows:].abs().max().item() == 0.0                           # tiles beyond num_m_tiles are not written


def test_mxfp8_linear_autograd(ops):
    torch.manual_seed(3)
    x = torch.randn(4, 96, 256, device="cuda").bfloat16().requires_grad_()
    w1 = (torch.randn(256, 256, device="cuda") * 0.05).requires_grad_()
    w2 = (torch.randn(128, 256, device="cuda") * 0.05).requires_grad_()
    y = ops.linear_multi(x, (w1, w2), "mxfp8")
    g = torch.randn_like(y)
    y.backward(g)
    x2 = x.detach().float().requires_grad_()
    wc = torch.cat((w1, w2)).detach().bfloat16().float().requires_grad_()
    want = ref.mxfp8_linear(x2.reshape(-1, 256), wc)
    assert rel(y.reshape(-1, 384), want) < 4e-3
    g2 = g.float().reshape(-1, 384)
    dx = ref.mxfp8_roundtrip(g2, -1) @ ref.mxfp8_roundtrip(wc.detach(), 0)
    assert rel(x.grad.reshape(-1, 256), dx) < 4e-3
    dw = g2.t() @ x2.detach().reshape(-1, 256)                           # weight gradient stays bf16 x bf16 -> fp32
    assert rel(torch.cat((w1.grad, w2.grad)), dw) < 1e-4


@pytest.mark.parametrize("top_k,experts,act", [(1, 8, "swiglu"), (2, 4, "relu2")])
def test_mxfp8_moe_experts(ops, top_k, experts, act):
    torch.manual_seed(4)
    m, d, h = 1000, 128, 256
    up_w = 2 * h if act == "swiglu" else h
    hidden = torch.randn(m, d, device="cuda").bfloat16().requires_grad_()
    logits = torch.randn(m, experts, device="cuda")
    logits[:, 1] = -1e4
    top_idx, gates, _ = ref.router_gates(logits, top_k, False)
    gates = gates.detach().requires_grad_()
    ups = [torch.randn(up_w, d, device="cuda").mul_(0.05).requires_grad_() for _ in range(experts)]
    downs = [torch.randn(d, h, device="cuda").mul_(0.05).requires_grad_() for _ in range(experts)]
    out = ops.moe_experts(hidden, top_idx, gates, ups, downs, None, None, act, "mxfp8", "mxfp8")
    g = torch.randn_like(out)
    out.backward(g)
    grads = [t.grad.clone() for t in [hidden, gates] + ups + downs]
    for t in [hidden, gates] + ups + downs:
        t.grad = None
    want = ops.moe_experts(hidden, top_idx, gates, ups, downs, None, None, act, "default", "default")
    want.backward(g)
    assert rel(out, want) < 1e-1                                          # fp8 against bf16: quantisation error only
    for a, b in zip(grads, [t.grad for t in [hidden, gates] + ups + downs]):
        assert rel(a, b) < 1.2e-1
    assert grads[2 + 1].abs().max().item() == 0.0
