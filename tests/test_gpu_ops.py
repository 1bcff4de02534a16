"""Model-operator kernels against plain PyTorch fp32 references (single GPU)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _C():
    import mccl_b200
    return mccl_b200._C


def _rel(a, b):
    return ((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-6)).item()


@pytest.fixture(params=["pair", "persistent"])
def gemm_kernel(request):
    """Runs a GEMM test once per kernel: CTA pairs (the default) and the one-CTA persistent kernel."""
    C = _C()
    C.set_gemm_kernel(request.param)
    yield request.param
    C.set_gemm_kernel("")


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 128), (4096, 512, 512), (4096, 1536, 512), (1000, 264, 192),
                                   (4096, 512, 2048), (130, 8, 64), (4096, 32000, 512), (4096, 2048, 512), (300, 2048, 64)])
def test_gemm_matches_fp32_reference(M, N, K, gemm_kernel):
    C = _C()
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    d, aux = C.gemm_bf16(a, b)
    torch.cuda.synchronize()
    assert C.gemm_error_flag() == 0
    ref = a.float() @ b.float().t()
    assert aux is None and d.dtype == torch.bfloat16
    assert _rel(d, ref) < 1e-2, _rel(d, ref)
    d32, _ = C.gemm_bf16(a, b, None, "none", True)
    assert _rel(d32, ref) < 1e-5 * max(1, K // 64), _rel(d32, ref)
    # accumulate into an fp32 output
    d32b, _ = C.gemm_bf16(a, b, None, "none", True, d32.clone(), True)
    assert _rel(d32b, 2 * ref) < 1e-4
    torch.cuda.synchronize()
    assert C.gemm_error_flag() == 0


@pytest.mark.parametrize("a_t,b_t", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (512, 384, 256), (2048, 512, 4096), (200, 72, 128)])
def test_gemm_mn_major_operands(a_t, b_t, M, N, K, gemm_kernel):
    """Operands stored [K, M] / [K, N] are read MN-major: same product, no transposed copy."""
    C = _C()
    torch.manual_seed(M * 3 + N * 5 + K)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    aa = a.t().contiguous() if a_t else a
    bb = b.t().contiguous() if b_t else b
    d, _ = C.gemm_bf16(aa, bb, None, "none", True, None, False, a_t, b_t)
    torch.cuda.synchronize()
    assert C.gemm_error_flag() == 0
    assert _rel(d, ref) < 1e-5 * max(1, K // 64), (_rel(d, ref), a_t, b_t)


@pytest.mark.parametrize("M,N,K", [(512, 256, 128), (1000, 2048, 192), (4096, 2048, 512)])
def test_gemm_epilogues_and_strides(M, N, K, gemm_kernel):
    C = _C()
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16() * 0.1
    bias = torch.randn(N, device="cuda")
    ref_z = a.float() @ b.float().t() + bias
    d, aux = C.gemm_bf16(a, b, bias, "none")
    assert _rel(d, ref_z) < 1e-2
    d, z = C.gemm_bf16(a, b, bias, "gelu")
    assert _rel(z, ref_z) < 1e-2 and _rel(d, F.gelu(ref_z)) < 1e-2
    d, z = C.gemm_bf16(a, b, None, "gelu")
    assert _rel(d, F.gelu(a.float() @ b.float().t())) < 1e-2
    # gelu_d: the second output is gelu'(z) instead of z
    d, dz = C.gemm_bf16(a, b, bias, "gelu_d")
    zz = ref_z.clone().requires_grad_(True)
    F.gelu(zz).sum().backward()
    assert _rel(d, F.gelu(ref_z)) < 1e-2 and _rel(dz, zz.grad) < 1e-2
    # residual added after the bias; multiplier applied to the product (the backward of a GELU)
    res = torch.randn(M, N, device="cuda").bfloat16()
    d, _ = C.gemm_bf16(a, b, bias, "none", False, None, False, False, False, res)
    assert _rel(d, ref_z + res.float()) < 1e-2
    mul = torch.randn(M, N, device="cuda").bfloat16()
    d, _ = C.gemm_bf16(a, b, None, "none", False, None, False, False, False, None, mul)
    assert _rel(d, (a.float() @ b.float().t()) * mul.float()) < 1e-2
    # row strides larger than K (views into wider buffers)
    wide_a = torch.randn(M, 3 * K, device="cuda").bfloat16()
    av = wide_a[:, K:2 * K]
    d, _ = C.gemm_bf16(av, b)
    assert _rel(d, av.float() @ b.float().t()) < 1e-2
    torch.cuda.synchronize()
    assert C.gemm_error_flag() == 0


@pytest.mark.parametrize("dim", [128, 512, 768, 2048])
@pytest.mark.parametrize("layernorm", [True, False])
def test_norm_forward_backward(dim, layernorm):
    C = _C()
    torch.manual_seed(dim)
    rows = 777
    x = (torch.randn(rows, dim, device="cuda") * 2 + 0.5).bfloat16()
    w = torch.randn(dim, device="cuda")
    b = torch.randn(dim, device="cuda") if layernorm else None
    dy = torch.randn(rows, dim, device="cuda").bfloat16()
    y, mean, rstd = C.norm_fwd(x, w, b, 1e-5)
    xr = x.float().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    if layernorm:
        br = b.clone().requires_grad_(True)
        yr = F.layer_norm(xr, (dim,), wr, br, 1e-5)
    else:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    assert _rel(y, yr) < 1e-2
    yr.backward(dy.float())
    dx, dw, db = C.norm_bwd(dy, x, w, mean, rstd, layernorm)
    assert _rel(dx, xr.grad) < 2e-2
    assert _rel(dw, wr.grad) < 1e-3
    if layernorm:
        assert _rel(db, br.grad) < 1e-3


def test_adamw_matches_reference():
    from mccl_b200.ops import reference
    C = _C()
    torch.manual_seed(0)
    n = 100_003
    p = torch.randn(n + 1, device="cuda")[:n - 3].contiguous()
    n = p.numel()
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    step = torch.zeros((), device="cuda")
    for s in range(1, 4):
        step.add_(1.0)
        C.adamw_flat(p, g, m, v, p16, 1e-2, 0.9, 0.999, 1e-8, 0.1, step, 1.0)
        pr, mr, vr = reference.adamw_step(pr, g, mr, vr, 1e-2, 0.9, 0.999, 1e-8, 0.1, s)
    assert _rel(p, pr) < 1e-5 and _rel(m, mr) < 1e-5 and _rel(v, vr) < 1e-4  # (1 - beta2) is rounded to fp32 in the kernel
    assert torch.equal(p16, p.bfloat16())


@pytest.mark.parametrize("T,V", [(64, 512), (300, 32000), (17, 1000)])
def test_cross_entropy_forward_backward(T, V):
    C = _C()
    torch.manual_seed(T)
    logits = (torch.randn(T, V, device="cuda") * 3).bfloat16()
    targets = torch.randint(0, V, (T,), device="cuda")
    ref_in = logits.float().requires_grad_(True)
    ref = F.cross_entropy(ref_in, targets)
    ref.backward()
    work = logits.clone()
    rows = C.ce_fwd_bwd(work, targets, 1.0 / T)
    assert abs(rows.mean().item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    assert _rel(work, ref_in.grad) < 2e-2


def test_transpose_cast_gelu_bwd():
    C = _C()
    cs = torch.randn(1000, 520, device="cuda").bfloat16()
    assert _rel(C.colsum_bf16(cs), cs.float().sum(0)) < 1e-5
    x = torch.randn(300, 520, device="cuda").bfloat16()
    assert torch.equal(C.transpose_bf16(x), x.t().contiguous())
    f = torch.randn(1001, device="cuda")[1:].contiguous() if False else torch.randn(1004, device="cuda")
    assert torch.equal(C.cast_bf16(f), f.bfloat16())
    z = torch.randn(64, 256, device="cuda").bfloat16()
    dy = torch.randn(64, 256, device="cuda").bfloat16()
    zr = z.float().requires_grad_(True)
    F.gelu(zr).backward(dy.float())
    assert _rel(C.gelu_bwd(dy, z), zr.grad) < 1e-2


def test_decoder_native_matches_torch_path():
    """Same weights, same batch: loss and gradients of the native operators vs stock PyTorch ops."""
    from mccl_b200.models import build_decoder
    torch.manual_seed(0)
    a = build_decoder("tiny", native=True).cuda()
    b = build_decoder("tiny", native=False).cuda()
    b.load_state_dict(a.state_dict())
    tok = torch.randint(0, a.cfg.vocab, (4, 65), device="cuda")
    la = a(tok[:, :-1], tok[:, 1:])
    lb = b(tok[:, :-1], tok[:, 1:])
    assert abs(la.item() - lb.item()) < 2e-2, (la.item(), lb.item())
    la.backward()
    lb.backward()
    worst = 0.0
    for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        denom = pb.grad.abs().max().clamp_min(1e-6)
        worst = max(worst, ((pa.grad - pb.grad).abs().max() / denom).item())
    assert worst < 8e-2, worst
    torch.cuda.synchronize()
    assert _C().gemm_error_flag() == 0


def test_direct_gradient_sinks_match_autograd():
    """Operators that write parameter gradients straight into preallocated fp32 buffers
    (what the training engine asks for) give the same gradients as the autograd path."""
    from mccl_b200.models import build_decoder
    torch.manual_seed(0)
    a = build_decoder("tiny", native=True).cuda()
    b = build_decoder("tiny", native=True).cuda()
    b.load_state_dict(a.state_dict())
    for p in a.parameters():
        p.grad = torch.zeros_like(p)
        p._grad_sink = p.grad
    tok = torch.randint(0, a.cfg.vocab, (4, 65), device="cuda")
    a(tok[:, :-1], tok[:, 1:]).backward()
    b(tok[:, :-1], tok[:, 1:]).backward()
    for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        denom = pb.grad.abs().max().clamp_min(1e-6)
        assert ((pa.grad - pb.grad).abs().max() / denom).item() < 1e-3, n


@pytest.mark.parametrize("with_pos", [True, False])
def test_embedding_forward_backward(with_pos):
    from mccl_b200 import ops
    torch.manual_seed(5)
    V, D, B, S = 300, 64, 3, 17
    tok = torch.randn(V, D, device="cuda", requires_grad=True)
    pos = torch.randn(S + 4, D, device="cuda", requires_grad=True) if with_pos else None
    ids = torch.randint(0, V, (B, S), device="cuda")
    ids[0, :4] = 7   # repeated ids: their gradients must add up
    y = ops.embedding(ids, tok, pos)
    ref = F.embedding(ids, tok.detach()) + (pos.detach()[:S] if with_pos else 0)
    assert y.dtype == torch.bfloat16 and y.shape == (B, S, D)
    assert _rel(y, ref) < 1e-2
    dy = torch.randn(B, S, D, device="cuda").bfloat16()
    y.backward(dy)
    tref = torch.zeros(V, D, device="cuda").index_add_(0, ids.reshape(-1), dy.float().reshape(-1, D))
    assert _rel(tok.grad, tref) < 1e-5
    if with_pos:
        pref = torch.zeros(S + 4, D, device="cuda")
        pref[:S] = dy.float().sum(0)
        assert _rel(pos.grad, pref) < 1e-5


@pytest.mark.parametrize("layernorm", [True, False])
def test_norm_backward_adds_residual_gradient(layernorm):
    C = _C()
    torch.manual_seed(3)
    rows, dim = 300, 512
    x = torch.randn(rows, dim, device="cuda").bfloat16()
    w = torch.randn(dim, device="cuda")
    b = torch.randn(dim, device="cuda") if layernorm else None
    dy = torch.randn(rows, dim, device="cuda").bfloat16()
    dres = torch.randn(rows, dim, device="cuda").bfloat16()
    _, mean, rstd = C.norm_fwd(x, w, b, 1e-5)
    dx0, dw0, _ = C.norm_bwd(dy, x, w, mean, rstd, layernorm)
    dx1, dw1, _ = C.norm_bwd(dy, x, w, mean, rstd, layernorm, None, None, False, dres)
    assert torch.equal(dw0, dw1)
    assert _rel(dx1, dx0.float() + dres.float()) < 1e-2


def test_norm_residual_function_matches_separate_add():
    from mccl_b200 import ops
    torch.manual_seed(4)
    x = torch.randn(64, 256, device="cuda").bfloat16().requires_grad_(True)
    w = torch.randn(256, device="cuda", requires_grad=True)
    b = torch.randn(256, device="cuda", requires_grad=True)
    y, xr = ops.norm_residual(x, w, b, 1e-5)
    out = (y * 2).float().sum() + (xr.float() * 3).sum()
    out.backward()
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = b.grad = None
    out2 = (ops.norm(x, w, b, 1e-5) * 2).float().sum() + (x.float() * 3).sum()
    out2.backward()
    assert _rel(gx, x.grad) < 1e-2 and _rel(gw, w.grad) < 1e-4


@pytest.mark.parametrize("with_residual", [True, False])
def test_fused_mlp_matches_fp32_reference(with_residual):
    """gelu(x W1^T + b1) W2^T + b2 (+ residual) as one autograd node: forward and every gradient against a plain
    fp32 PyTorch computation of the same block (the input-gradient GEMM of the second layer multiplies by
    gelu'(z) in its epilogue)."""
    from mccl_b200 import ops
    torch.manual_seed(3)
    T, D, FF = 256, 128, 512
    x = (torch.randn(T, D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    res = (torch.randn(T, D, device="cuda") * 0.5).bfloat16().requires_grad_(True) if with_residual else None
    w1 = (torch.randn(FF, D, device="cuda") * 0.05).requires_grad_(True)
    b1 = (torch.randn(FF, device="cuda") * 0.1).requires_grad_(True)
    w2 = (torch.randn(D, FF, device="cuda") * 0.05).requires_grad_(True)
    b2 = (torch.randn(D, device="cuda") * 0.1).requires_grad_(True)
    y = ops.mlp_gelu(x, w1, b1, w2, b2, residual=res)
    dy = (torch.randn(T, D, device="cuda") * 0.1).bfloat16()
    y.backward(dy)
    got = [x.grad, w1.grad, b1.grad, w2.grad, b2.grad] + ([res.grad] if with_residual else [])
    # fp32 reference on the bf16-rounded inputs and weights
    xr = x.detach().float().requires_grad_(True)
    rr = res.detach().float().requires_grad_(True) if with_residual else None
    w1r, b1r = w1.detach().bfloat16().float().requires_grad_(True), b1.detach().clone().requires_grad_(True)
    w2r, b2r = w2.detach().bfloat16().float().requires_grad_(True), b2.detach().clone().requires_grad_(True)
    yr = F.gelu(xr @ w1r.t() + b1r) @ w2r.t() + b2r
    if with_residual:
        yr = yr + rr
    yr.backward(dy.float())
    assert _rel(y, yr) < 2e-2
    want = [xr.grad, w1r.grad, b1r.grad, w2r.grad, b2r.grad] + ([rr.grad] if with_residual else [])
    for g, w, name in zip(got, want, ["dx", "dw1", "db1", "dw2", "db2", "dres"]):
        assert _rel(g, w) < 2e-2, (name, _rel(g, w))
    assert _C().gemm_error_flag() == 0


@pytest.mark.parametrize("B,S,H", [(2, 128, 2), (2, 256, 4), (16, 256, 8)])
def test_causal_attention_forward_backward(B, S, H):
    """The tcgen05 attention kernels (head dimension 64) against a plain fp32 PyTorch computation: softmax(q k^T / 8
    + causal mask) v on the q, k, v slices of the fused projection's output, and the gradient of that whole tensor."""
    from mccl_b200 import ops
    torch.manual_seed(B * 1000 + S + H)
    D = 64
    qkv = (torch.randn(B, S, 3 * H * D, device="cuda") * 0.7).bfloat16().requires_grad_(True)
    out = ops.causal_attention(qkv, H)
    assert out.shape == (B, S, H * D)
    d_out = (torch.randn(B, S, H * D, device="cuda") * 0.5).bfloat16()
    out.backward(d_out)
    ref_in = qkv.detach().float().requires_grad_(True)
    q, k, v = (t.transpose(1, 2) for t in ref_in.view(B, S, 3, H, D).unbind(2))      # [B, H, S, D]
    scores = (q @ k.transpose(-1, -2)) / (D ** 0.5)
    mask = torch.ones(S, S, device="cuda", dtype=torch.bool).tril()
    probs = scores.masked_fill(~mask, float("-inf")).softmax(-1)
    ref = (probs @ v).transpose(1, 2).reshape(B, S, H * D)
    ref.backward(d_out.float())
    assert _rel(out, ref) < 2e-2, _rel(out, ref)
    got, want = qkv.grad.view(B, S, 3, H, D), ref_in.grad.view(B, S, 3, H, D)
    for t, name in enumerate(("dq", "dk", "dv")):
        assert _rel(got[:, :, t], want[:, :, t]) < 2e-2, (name, _rel(got[:, :, t], want[:, :, t]))
    assert _C().gemm_error_flag() == 0
