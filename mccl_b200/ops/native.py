"""autograd Functions over the native kernels (CUDA tensors only)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _C


def _bf16_weight(weight: torch.Tensor) -> torch.Tensor:
    """bf16 copy of an fp32 parameter: the trainer keeps one up to date (`_bf16`), else cast now."""
    w16 = getattr(weight, "_bf16", None)
    if w16 is not None:
        return w16
    if weight.dtype == torch.bfloat16:
        return weight
    return _C.cast_bf16(weight.detach().contiguous())


def _sink(p: torch.Tensor):
    """fp32 buffer a trainer wants this parameter's gradient written into (or None)."""
    return getattr(p, "_grad_sink", None)


def _notify(p: torch.Tensor) -> None:
    """Tells the trainer that p's gradient is complete (it was written in place, so autograd's
    own accumulation hook will not fire).  Parameters whose gradient has further contributions
    from autograd (tied embeddings) are marked `_shared_grad` and notified by autograd instead."""
    if getattr(p, "_shared_grad", False):
        return
    cb = getattr(p, "_grad_ready", None)
    if cb is not None:
        cb()


# Weight-gradient GEMMs have no consumer until the gradient is reduced or applied, so a trainer can give them a
# stream of their own: they then run beside the input-gradient chain and fill the SMs its small kernels leave idle.
_wgrad = {"stream": None, "pending": False, "side_ctas": 0, "main_ctas": 0}
_SIDE_COLSUM = __import__("os").environ.get("MCCL_SIDE_COLSUM", "1") != "0"


def set_wgrad_stream(stream, main_ctas: int = 0, side_ctas: int = 0) -> None:
    """Side stream for weight-gradient GEMMs that write into a trainer's gradient buffer (None: current stream).
    main_ctas / side_ctas: CTA caps of the GEMMs on the caller's stream and on the side stream while it is set
    (0: no cap); with caps that add up to the SM count a GEMM of one stream never waits for CTAs of the other."""
    _wgrad["stream"] = stream
    _wgrad["pending"] = False
    _wgrad["main_ctas"], _wgrad["side_ctas"] = main_ctas, side_ctas


def mark_wgrad_pending() -> None:
    """A trainer queued work of its own on the weight-gradient stream."""
    _wgrad["pending"] = True


def join_wgrad(stream=None) -> None:
    """Makes ``stream`` (default: the current one) wait for the weight gradients queued on the side stream."""
    s = _wgrad["stream"]
    if s is not None and _wgrad["pending"]:
        (stream if stream is not None else torch.cuda.current_stream()).wait_stream(s)


def _wgrad_gemm(a_mat: torch.Tensor, b_mat: torch.Tensor, sink: torch.Tensor) -> None:
    """sink += a_mat^T . b_mat (both [tokens, features]) on the weight-gradient stream."""
    s = _wgrad["stream"]
    if s is None:
        _C.gemm_bf16(a_mat, b_mat, None, "none", True, sink, True, True, True)
        return
    s.wait_stream(torch.cuda.current_stream())
    if _wgrad["side_ctas"]:
        _C.set_gemm_cta_limit(_wgrad["side_ctas"])
    with torch.cuda.stream(s):
        _C.gemm_bf16(a_mat, b_mat, None, "none", True, sink, True, True, True)
    if _wgrad["side_ctas"]:
        _C.set_gemm_cta_limit(_wgrad["main_ctas"])
    a_mat.record_stream(s)
    b_mat.record_stream(s)
    _wgrad["pending"] = True


def _norm_param_grads(dyc, x, weight, mean, rstd, layernorm, wsink, bsink) -> bool:
    """dw / db of a norm on the weight-gradient stream; False when there is none (the caller then computes them in line)."""
    s = _wgrad["stream"] if _SIDE_COLSUM else None
    if s is None:
        return False
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        _C.norm_bwd(dyc, x, weight, mean, rstd, layernorm, wsink, bsink, True, None, 2)
    for t in (dyc, x, mean, rstd):
        t.record_stream(s)
    _wgrad["pending"] = True
    return True


def _wgrad_colsum(src: torch.Tensor, sink: torch.Tensor) -> None:
    """sink += column sums of src (a bias gradient), on the weight-gradient stream."""
    s = _wgrad["stream"] if _SIDE_COLSUM else None
    if s is None:
        _C.colsum_bf16(src, sink, True)
        return
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        _C.colsum_bf16(src, sink, True)
    src.record_stream(s)
    _wgrad["pending"] = True


def _gemm_ok(m: int, n: int, k: int) -> bool:
    return k % 64 == 0 and n % 8 == 0 and m > 0


class LinearFn(torch.autograd.Function):
    """y = act(x @ W^T + b); W [N, K] fp32 master, x [..., K] bf16."""

    @staticmethod
    def forward(ctx, x, weight, bias, act, residual=None):
        K, N = weight.shape[1], weight.shape[0]
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        w16 = _bf16_weight(weight)
        ctx.act, ctx.has_bias, ctx.native = act, bias is not None, _gemm_ok(M, N, K)
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, N)
            if not res2.is_contiguous():
                res2 = res2.contiguous()
        ctx.has_residual = residual is not None
        if ctx.native:
            y, z = _C.gemm_bf16(x2, w16, bias, act, False, None, False, False, False, res2)
        else:
            z = F.linear(x2, w16, None if bias is None else bias.to(x2.dtype))
            y = F.gelu(z) if act == "gelu" else z
            z = z if act == "gelu" else None
            if res2 is not None:
                y = y + res2
        ctx.save_for_backward(x2, w16, z if z is not None else x2.new_empty(0))
        ctx.weight, ctx.bias = weight, bias
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, w16, z = ctx.saved_tensors
        weight = ctx.weight
        N, K = w16.shape
        M = x2.shape[0]
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dz = _C.gelu_bwd(dy2, z) if ctx.act == "gelu" else dy2
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            if _gemm_ok(M, K, N):
                # dx[M,K] = dz[M,N] · W[N,K]: W is the B operand stored [contraction, K], read MN-major
                dx, _ = _C.gemm_bf16(dz, w16, None, "none", False, None, False, False, True)
            else:
                dx = dz @ w16
            dx = dx.view(*dy.shape[:-1], K)
        if ctx.needs_input_grad[1]:
            sink = _sink(weight)
            if _gemm_ok(N, K, M) and N % 8 == 0:
                # dW[N,K] = dz^T · x: both operands stored [tokens, features], read MN-major
                if sink is not None:
                    _wgrad_gemm(dz, x2, sink)
                    _notify(weight)
                else:
                    dw, _ = _C.gemm_bf16(dz, x2, None, "none", True, None, False, True, True)
            else:
                dw = (dz.t() @ x2).float()
        if ctx.has_bias and ctx.needs_input_grad[2]:
            bsink = _sink(ctx.bias)
            if N % 8 == 0:
                if bsink is not None:
                    _wgrad_colsum(dz, bsink)
                    _notify(ctx.bias)
                else:
                    db = _C.colsum_bf16(dz)
            else:
                db = dz.sum(0, dtype=torch.float32)
        dres = dy if ctx.has_residual else None
        return dx, dw, db, None, dres


class MlpGeluFn(torch.autograd.Function):
    """y = gelu(x @ W1^T + b1) @ W2^T + b2 (+ residual) as one autograd node, so that backward can fuse across
    the two layers: the first GEMM's epilogue saves gelu'(z) next to gelu(z) (they share the erf), and the
    input-gradient GEMM of the second layer multiplies by it in its epilogue and writes dz directly, so there is
    no separate GELU-backward pass over the [tokens, d_ff] tensor.  (Evaluating erf and exp in the backward
    epilogue instead was measured slower than the separate kernel: four epilogue warps per SM are too few for it.)"""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual=None):
        D, FF = w1.shape[1], w1.shape[0]
        x2 = x.reshape(-1, D)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        w1_16, w2_16 = _bf16_weight(w1), _bf16_weight(w2)
        h, z = _C.gemm_bf16(x2, w1_16, b1, "gelu_d")   # z holds gelu'(pre-activation)
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, w2.shape[0])
            if not res2.is_contiguous():
                res2 = res2.contiguous()
        y, _ = _C.gemm_bf16(h, w2_16, b2, "none", False, None, False, False, False, res2)
        ctx.save_for_backward(x2, w1_16, w2_16, z, h)
        ctx.params = (w1, b1, w2, b2)
        ctx.has_residual = residual is not None
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1_16, w2_16, z, h = ctx.saved_tensors
        w1, b1, w2, b2 = ctx.params
        dy2 = dy.reshape(-1, w2_16.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        # second layer: dz = (dy . W2) * gelu'(pre-activation) in one kernel; dW2 = dy^T . h; db2 = column sums of dy
        dz, _ = _C.gemm_bf16(dy2, w2_16, None, "none", False, None, False, False, True, None, z)
        # the input gradient first: every reader of this node's weights is queued before a parameter is reported
        # complete (a trainer may start that parameter's optimizer update on another stream as soon as it is)
        dx = None
        if ctx.needs_input_grad[0]:
            dx, _ = _C.gemm_bf16(dz, w1_16, None, "none", False, None, False, False, True)
            dx = dx.view(*dy.shape[:-1], w1_16.shape[1])
        grads = {}
        for name, (w, a_mat, b_mat) in (("w2", (w2, dy2, h)), ("w1", (w1, dz, x2))):
            sink = _sink(w)
            if sink is not None:
                _wgrad_gemm(a_mat, b_mat, sink)
                _notify(w)
                grads[name] = None
            else:
                grads[name], _ = _C.gemm_bf16(a_mat, b_mat, None, "none", True, None, False, True, True)
        for name, (b, src) in (("b2", (b2, dy2)), ("b1", (b1, dz))):
            if b is None:
                grads[name] = None
                continue
            bsink = _sink(b)
            if bsink is not None:
                _wgrad_colsum(src, bsink)
                _notify(b)
                grads[name] = None
            else:
                grads[name] = _C.colsum_bf16(src)
        return dx, grads["w1"], grads["b1"], grads["w2"], grads["b2"], (dy if ctx.has_residual else None)


class CausalAttentionFn(torch.autograd.Function):
    """Causal self-attention on the output of the fused QKV projection, viewed as [B, S, 3, H, 64]: one kernel
    forward, one backward, both on the tcgen05 tensor cores; the gradient comes back for the whole qkv tensor, so
    no slices, transposes or concatenations surround the kernels."""

    @staticmethod
    def forward(ctx, qkv, scale):
        q5 = qkv if qkv.is_contiguous() else qkv.contiguous()
        o, lse = _C.attn_fwd(q5, scale)
        ctx.save_for_backward(q5, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q5, o, lse = ctx.saved_tensors
        d = d_o if d_o.is_contiguous() else d_o.contiguous()
        return _C.attn_bwd(q5, o, d, lse, ctx.scale), None


class NormFn(torch.autograd.Function):
    """LayerNorm (bias given) or RMSNorm (bias None) over the last dimension; fp32 weight / bias."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        xc = x if x.is_contiguous() else x.contiguous()
        y, mean, rstd = _C.norm_fwd(xc, weight, bias, eps)
        ctx.save_for_backward(xc, weight, mean, rstd)
        ctx.layernorm = bias is not None
        ctx.weight, ctx.bias = weight, bias
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, mean, rstd = ctx.saved_tensors
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        wsink, bsink = _sink(ctx.weight), (_sink(ctx.bias) if ctx.bias is not None else None)
        if wsink is not None and (not ctx.layernorm or bsink is not None):
            # the sinks were zeroed at the start of the step; the kernel adds into them
            side = _norm_param_grads(dyc, x, weight, mean, rstd, ctx.layernorm, wsink, bsink)
            dx, _, _ = _C.norm_bwd(dyc, x, weight, mean, rstd, ctx.layernorm, wsink, bsink, True, None, 1 if side else 3)
            _notify(ctx.weight)
            if ctx.bias is not None:
                _notify(ctx.bias)
            return dx, None, None, None
        dx, dw, db = _C.norm_bwd(dyc, x, weight, mean, rstd, ctx.layernorm)
        return dx, dw, db, None


class NormResidualFn(torch.autograd.Function):
    """Norm of a tensor that also continues as a residual: returns ``(norm(x), x)``.  In backward the
    gradient that comes back along the residual is added inside the norm-backward kernel (before its
    single rounding to bf16) instead of by a separate add kernel."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        xc = x if x.is_contiguous() else x.contiguous()
        y, mean, rstd = _C.norm_fwd(xc, weight, bias, eps)
        ctx.save_for_backward(xc, weight, mean, rstd)
        ctx.layernorm = bias is not None
        ctx.weight, ctx.bias = weight, bias
        return y, xc.view_as(xc)

    @staticmethod
    def backward(ctx, dy, dres):
        x, weight, mean, rstd = ctx.saved_tensors
        if dy is None:
            return dres, None, None, None
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        add = None if dres is None else (dres if dres.is_contiguous() else dres.contiguous())
        wsink, bsink = _sink(ctx.weight), (_sink(ctx.bias) if ctx.bias is not None else None)
        if wsink is not None and (not ctx.layernorm or bsink is not None):
            side = _norm_param_grads(dyc, x, weight, mean, rstd, ctx.layernorm, wsink, bsink)
            dx, _, _ = _C.norm_bwd(dyc, x, weight, mean, rstd, ctx.layernorm, wsink, bsink, True, add, 1 if side else 3)
            _notify(ctx.weight)
            if ctx.bias is not None:
                _notify(ctx.bias)
            return dx, None, None, None
        dx, dw, db = _C.norm_bwd(dyc, x, weight, mean, rstd, ctx.layernorm, None, None, False, add)
        return dx, dw, db, None


class LinearCrossEntropyFn(torch.autograd.Function):
    """mean CE(h @ W^T, targets).  The backward of the loss with respect to the logits is
    produced in the same pass that computes the loss, in place of the logits, assuming the
    loss is what ``backward()`` is called on (upstream gradient 1)."""

    @staticmethod
    def forward(ctx, h, weight, targets):
        T, D = h.shape
        V = weight.shape[0]
        hc = h if h.is_contiguous() else h.contiguous()
        w16 = _bf16_weight(weight)
        if _gemm_ok(T, V, D):
            logits, _ = _C.gemm_bf16(hc, w16)
        else:
            logits = F.linear(hc, w16)
        loss_rows = _C.ce_fwd_bwd(logits, targets.contiguous(), 1.0 / T)
        ctx.save_for_backward(hc, w16, logits)   # logits now hold d(loss)/d(logits)
        ctx.weight = weight
        return loss_rows.mean()

    @staticmethod
    def backward(ctx, gout):
        h, w16, dlogits = ctx.saved_tensors
        weight = ctx.weight
        T, D = h.shape
        V = w16.shape[0]
        dh = dw = None
        if ctx.needs_input_grad[0]:
            if _gemm_ok(T, D, V):
                dh, _ = _C.gemm_bf16(dlogits, w16, None, "none", False, None, False, False, True)
            else:
                dh = dlogits @ w16
        if ctx.needs_input_grad[1]:
            sink = _sink(weight)
            if _gemm_ok(V, D, T) and V % 8 == 0:
                if sink is not None:
                    _wgrad_gemm(dlogits, h, sink)
                    _notify(weight)
                else:
                    dw, _ = _C.gemm_bf16(dlogits, h, None, "none", True, None, False, True, True)
            else:
                dw = (dlogits.t() @ h).float()
        return dh, dw, None


class EmbeddingFn(torch.autograd.Function):
    """bf16(tok[ids] + pos[position]) in one kernel; the backward adds the output gradient into the
    fp32 gradient buffers of both tables (the trainer's sinks when there are any) with vector atomics,
    so no sort, no dense zero-filled intermediate and no autograd accumulation step is needed."""

    @staticmethod
    def forward(ctx, ids, tok, pos, seq):
        flat = ids.reshape(-1).contiguous()
        y = _C.embed_fwd(flat, tok.detach(), None if pos is None else pos.detach(), seq)
        ctx.save_for_backward(flat)
        ctx.tok, ctx.pos, ctx.seq = tok, pos, seq
        return y.view(*ids.shape, tok.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        tok, pos, seq = ctx.tok, ctx.pos, ctx.seq
        dyc = dy.reshape(-1, tok.shape[1])
        if not dyc.is_contiguous():
            dyc = dyc.contiguous()
        tsink = _sink(tok)
        psink = _sink(pos) if pos is not None else None
        dtok = tsink if tsink is not None else torch.zeros_like(tok, dtype=torch.float32)
        dpos = None
        if pos is not None:
            dpos = psink if psink is not None else torch.zeros_like(pos, dtype=torch.float32)
        _C.embed_bwd(flat, dyc, dtok, dpos, seq)
        # this is the last contribution to a tied table's gradient, so it is the one that reports it
        for p, sink in ((tok, tsink), (pos, psink)):
            if p is not None and sink is not None:
                cb = getattr(p, "_grad_ready", None)
                if cb is not None:
                    cb()
        return None, (None if tsink is not None else dtok), (None if pos is None or psink is not None else dpos), None

