"""Differentiable ops: each CUDA op is a ``torch.autograd.Function`` over the
hand-written sm_100a kernels; each has a PyTorch-CPU twin so the same model
code runs on the CPU backend (the default backend and correctness oracle, as
in the reference: crates/incin/src/lib.rs:143-167).

Parameter gradients are not returned through autograd.  They are accumulated
in fp32 straight into ``param.main_grad`` (a view of the flat gradient buffer
owned by :class:`incin_b200.optim.flat.ParamStore`) by the weight-gradient GEMM
(split-K, fp32 atomics), the column-sum kernel and the norm backward kernels.
This keeps gradients in one contiguous buffer that the fused data-parallel
reduce + AdamW kernel consumes bucket by bucket, and it makes tied weights and
gradient accumulation free.  ``param._grad_ready`` (if set) is called once the
parameter's gradient for this backward pass is complete.

The residual stream is threaded through ``*_fork`` ops and GEMM epilogues so
that no elementwise add is left to autograd: ``layernorm_fork`` returns
``(x, LN(x))`` and its backward fuses ``dLN + d_residual`` into one kernel.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as TF

from .. import _native as nat
from . import gemm as G
from . import kernels as K

ACT = {None: nat.ACT_NONE, "none": nat.ACT_NONE, "gelu": nat.ACT_GELU, "silu": nat.ACT_SILU}
_DACT = {nat.ACT_GELU: nat.ACT_DGELU, nat.ACT_SILU: nat.ACT_DSILU}

# CTAs the compute GEMMs may use; lowered while a communication kernel shares the GPU
_max_ctas = 0


def set_compute_ctas(n: int) -> None:
    global _max_ctas
    _max_ctas = int(n)


def main_grad(p: torch.Tensor) -> torch.Tensor:
    g = getattr(p, "main_grad", None)
    if g is None:
        g = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        p.main_grad = g
    return g


def _ready(p: torch.Tensor) -> None:
    cb = getattr(p, "_grad_ready", None)
    if cb is not None:
        cb(p)


def _nat(t: torch.Tensor) -> bool:
    """True when the hand-written sm_100a kernels take this tensor (CUDA + bf16); other dtypes and the CPU
    use the PyTorch twin of the op."""
    return t.is_cuda and t.dtype == torch.bfloat16


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


# --------------------------------------------------------------------------------------------- linear
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, residual, act, defer_bias_grad=False):
        x = _c(x)
        ctx.defer_bias = defer_bias_grad
        aux = None
        if act != nat.ACT_NONE:
            aux = torch.empty(*x.shape[:-1], w.shape[0], dtype=torch.bfloat16, device=x.device)
        y = G.mm_nt(x, w, bias=b, residual=_c(residual) if residual is not None else None, act=act, aux=aux,
                    max_ctas=_max_ctas)
        ctx.save_for_backward(x, w, aux)
        ctx.has_bias = b is not None
        ctx.bias = b
        ctx.act = act
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, aux = ctx.saved_tensors
        dy = _c(dy)
        dpre = K.act_bwd(dy, aux, ctx.act) if ctx.act != nat.ACT_NONE else dy
        if w.requires_grad:
            G.mm_tn_accum(dpre, x, main_grad(w), max_ctas=_max_ctas)
        own_bias = ctx.has_bias and ctx.bias.requires_grad and not ctx.defer_bias
        if own_bias:
            K.colsum_accum(dpre, main_grad(ctx.bias))
        dx = G.mm_nn(dpre, w, max_ctas=_max_ctas) if ctx.needs_input_grad[0] else None
        # A ready callback may launch the data-parallel update, which overwrites w on another stream: it is
        # called only after the last kernel that reads w (the data-gradient product above) has been enqueued.
        if w.requires_grad:
            _ready(w)
        if own_bias:
            _ready(ctx.bias)
        return dx, None, None, (dy if ctx.has_res else None), None, None


class _LinearF32Acc(torch.autograd.Function):
    """Linear for fp16 tensors and, under ``MathMode.FAST``, fp32 tensors (multiplied as tf32) on the same tcgen05
    kernel as the bf16 path: fp32 accumulation and fp32 output, rounded once to the input type.  Gradients return
    through autograd; the transposed operands the two backward products need are materialised (these types are the
    breadth path, bf16 is the tuned one)."""

    @staticmethod
    def forward(ctx, x, w, b):
        x2 = _c(x).reshape(-1, x.shape[-1])
        y = G.mm_nt_f32out(x2, _c(w))
        if b is not None:
            y += b.float()
        ctx.save_for_backward(x2, w)
        ctx.has_bias = b is not None
        ctx.shape = x.shape
        return y.to(x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _c(dy).reshape(-1, dy.shape[-1])
        unit = 8 if dy2.dtype == torch.float16 else 4
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            if dy2.shape[1] % unit == 0:
                dx = G.mm_nt_f32out(dy2, w.t().contiguous()).to(dy.dtype)
            else:
                dx = dy2 @ w
            dx = dx.reshape(ctx.shape)
        if ctx.needs_input_grad[1]:
            if dy2.shape[0] % unit == 0:
                dw = G.mm_nt_f32out(dy2.t().contiguous(), x2.t().contiguous()).to(w.dtype)
            else:
                dw = dy2.t() @ x2
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def _f32acc_native(x: torch.Tensor, w: torch.Tensor) -> bool:
    """fp16 always, fp32 when the execution policy allows fast math (tf32); rows must start on 16-byte boundaries."""
    if not (x.is_cuda and x.dtype == w.dtype and x.dim() >= 1 and w.dim() == 2):
        return False
    if x.dtype == torch.float16:
        return x.shape[-1] % 8 == 0
    if x.dtype == torch.float32:
        from ..core.policy import MathMode, current_policy
        return current_policy().math == MathMode.FAST and x.shape[-1] % 4 == 0
    return False


def linear(x, w, b=None, *, act=None, residual=None, defer_bias_grad: bool = False):
    """``act(x @ w^T + b) + residual`` with everything fused into the GEMM epilogue on CUDA.
    ``defer_bias_grad``: the bias gradient (column sums of this op's output gradient) is produced by the norm that
    consumes the output (``layernorm_fork(..., bias_of_input=b)``) instead of by a launch of its own."""
    if _nat(x):
        return _Linear.apply(x, w, b, residual, ACT[act], defer_bias_grad and act is None)
    y = _LinearF32Acc.apply(x, w, b) if _f32acc_native(x, w) else TF.linear(x, w, b)
    if act == "gelu":
        y = TF.gelu(y)
    elif act == "silu":
        y = TF.silu(y)
    return y if residual is None else y + residual


class _MLP(torch.autograd.Function):
    """y = act(x W1^T + b1) W2^T + b2 + residual; the activation backward rides in the dgrad GEMM epilogue."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual, act, defer_b2_grad=False):
        x = _c(x)
        ctx.defer_b2 = defer_b2_grad
        pre = torch.empty(*x.shape[:-1], w1.shape[0], dtype=torch.bfloat16, device=x.device)
        h = G.mm_nt(x, w1, bias=b1, act=act, aux=pre, max_ctas=_max_ctas)
        y = G.mm_nt(h, w2, bias=b2, residual=_c(residual) if residual is not None else None, max_ctas=_max_ctas)
        ctx.save_for_backward(x, w1, w2, pre, h)
        ctx.b1, ctx.b2, ctx.act, ctx.has_res = b1, b2, act, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w1, w2, pre, h = ctx.saved_tensors
        dy = _c(dy)
        G.mm_tn_accum(dy, h, main_grad(w2), max_ctas=_max_ctas)
        own_b2 = ctx.b2 is not None and not ctx.defer_b2
        if own_b2:
            K.colsum_accum(dy, main_grad(ctx.b2))
        dpre = G.mm_nn(dy, w2, act=_DACT[ctx.act], aux=pre, max_ctas=_max_ctas)
        # ready callbacks come after the last enqueued reader of each weight (they may start its update)
        _ready(w2)
        if own_b2:
            _ready(ctx.b2)
        G.mm_tn_accum(dpre, x, main_grad(w1), max_ctas=_max_ctas)
        if ctx.b1 is not None:
            K.colsum_accum(dpre, main_grad(ctx.b1))
        dx = G.mm_nn(dpre, w1, max_ctas=_max_ctas) if ctx.needs_input_grad[0] else None
        _ready(w1)
        if ctx.b1 is not None:
            _ready(ctx.b1)
        return dx, None, None, None, None, (dy if ctx.has_res else None), None, None


def mlp(x, w1, b1, w2, b2, *, act="gelu", residual=None, defer_b2_grad: bool = False):
    """``defer_b2_grad``: the gradient of ``b2`` is produced by the norm that consumes the output (see :func:`linear`)."""
    if _nat(x):
        return _MLP.apply(x, w1, b1, w2, b2, residual, ACT[act], defer_b2_grad and b2 is not None)
    h = TF.linear(x, w1, b1)
    h = TF.gelu(h) if act == "gelu" else TF.silu(h)
    y = TF.linear(h, w2, b2)
    return y if residual is None else y + residual


# --------------------------------------------------------------------------------------------- norms
class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, b, eps, fork, bias_of_input=None):
        x = _c(x)
        y, mean, rstd = K.layernorm_fwd(x, g, b, eps)
        ctx.save_for_backward(x, g, mean, rstd)
        ctx.b, ctx.fork = b, fork
        ctx.in_bias = bias_of_input if (bias_of_input is not None and bias_of_input.requires_grad) else None
        if fork:
            return x.view_as(x), y
        return y

    @staticmethod
    def backward(ctx, *grads):
        x, g, mean, rstd = ctx.saved_tensors
        if ctx.fork:
            dxid, dy = grads
        else:
            dxid, dy = None, grads[0]
        if dy is None:  # normalised branch unused: only the identity gradient flows
            if ctx.in_bias is not None and dxid is not None:
                K.colsum_accum(_c(dxid), main_grad(ctx.in_bias))
                _ready(ctx.in_bias)
            return dxid, None, None, None, None, None
        dg = main_grad(g) if g.requires_grad else None
        db = main_grad(ctx.b) if (ctx.b is not None and ctx.b.requires_grad) else None
        # the gradient this op returns is the output gradient of the linear layer in front of it: its column sums are
        # that layer's bias gradient and come out of the same pass
        dx = K.layernorm_bwd(_c(dy), x, g, mean, rstd, _c(dxid) if dxid is not None else None, dg, db,
                             main_grad(ctx.in_bias) if ctx.in_bias is not None else None)
        if dg is not None:
            _ready(g)
        if db is not None:
            _ready(ctx.b)
        if ctx.in_bias is not None:
            _ready(ctx.in_bias)
        return dx, None, None, None, None, None


def layer_norm(x, g, b=None, eps: float = 1e-5, *, bias_of_input=None):
    """``bias_of_input``: the bias of the linear layer that produced ``x`` (called with ``defer_bias_grad``); its
    gradient is accumulated by this op's backward."""
    if _nat(x):
        return _LayerNorm.apply(x, g, b, eps, False, bias_of_input)
    return TF.layer_norm(x, (x.shape[-1],), g, b, eps)


def layernorm_fork(x, g, b=None, eps: float = 1e-5, *, bias_of_input=None):
    """Returns ``(x, layer_norm(x))``; the backward adds both incoming gradients in the LN kernel (and accumulates the
    gradient of ``bias_of_input``, see :func:`layer_norm`)."""
    if _nat(x):
        return _LayerNorm.apply(x, g, b, eps, True, bias_of_input)
    return x, TF.layer_norm(x, (x.shape[-1],), g, b, eps)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, eps, fork):
        x = _c(x)
        y, rstd = K.rmsnorm_fwd(x, g, eps)
        ctx.save_for_backward(x, g, rstd)
        ctx.fork = fork
        if fork:
            return x.view_as(x), y
        return y

    @staticmethod
    def backward(ctx, *grads):
        x, g, rstd = ctx.saved_tensors
        if ctx.fork:
            dxid, dy = grads
        else:
            dxid, dy = None, grads[0]
        if dy is None:
            return dxid, None, None, None
        dg = main_grad(g) if g.requires_grad else None
        dx = K.rmsnorm_bwd(_c(dy), x, g, rstd, _c(dxid) if dxid is not None else None, dg)
        if dg is not None:
            _ready(g)
        return dx, None, None, None


def _rms_cpu(x, g, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * g.float()).to(x.dtype)


def rms_norm(x, g, eps: float = 1e-5):
    if _nat(x):
        return _RMSNorm.apply(x, g, eps, False)
    return _rms_cpu(x, g, eps)


def rmsnorm_fork(x, g, eps: float = 1e-5):
    if _nat(x):
        return _RMSNorm.apply(x, g, eps, True)
    return x, _rms_cpu(x, g, eps)


# --------------------------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, wte, wpe):
        tokens = _c(tokens)
        ctx.save_for_backward(tokens)
        ctx.wte, ctx.wpe = wte, wpe
        return K.embedding_fwd(tokens, wte, wpe)

    @staticmethod
    def backward(ctx, dout):
        (tokens,) = ctx.saved_tensors
        wte, wpe = ctx.wte, ctx.wpe
        from ..core.policy import Determinism, current_policy
        if current_policy().determinism is Determinism.REQUIRED and not torch.cuda.is_current_stream_capturing():
            # fixed summation order: sort by token, one block per distinct token (not capturable: the number of
            # distinct tokens is read back to size the launch)
            from .tensor_ops import embedding_bwd_deterministic
            embedding_bwd_deterministic(_c(dout), tokens, main_grad(wte), main_grad(wpe) if wpe is not None else None,
                                        tokens.shape[-1])
        else:
            K.embedding_bwd(_c(dout), tokens, main_grad(wte), main_grad(wpe) if wpe is not None else None)
        _ready(wte)
        if wpe is not None:
            _ready(wpe)
        return None, None, None


def embedding(tokens, wte, wpe=None):
    """``wte[tokens] + wpe[arange(T)]`` (learned positions optional)."""
    if _nat(wte):
        return _Embedding.apply(tokens, wte, wpe)
    out = TF.embedding(tokens, wte)
    if wpe is not None:
        out = out + wpe[: tokens.shape[1]]
    return out


# --------------------------------------------------------------------------------------------- loss
class _CrossEntropy(torch.autograd.Function):
    """Mean softmax cross-entropy over rows; the backward overwrites the logits buffer with its gradient."""

    @staticmethod
    def forward(ctx, logits, targets, V):
        l2 = logits.view(-1, logits.shape[-1])
        t = _c(targets.view(-1))
        loss_rows, lse = K.xent_fwd(l2, t, V)
        ctx.save_for_backward(l2, t, lse)
        ctx.V, ctx.shape = V, logits.shape
        return K.mean_f32(loss_rows)

    @staticmethod
    def backward(ctx, dloss):
        l2, t, lse = ctx.saved_tensors
        K.xent_bwd_(l2, t, lse, _c(dloss.float()), 1.0 / l2.shape[0], ctx.V)
        return l2.view(ctx.shape), None, None


class _LinearCrossEntropy(torch.autograd.Function):
    """``mean CE(x @ w^T, targets)`` as one op: the logits are produced by the GEMM, turned into per-row losses AND
    into their own gradient by one kernel (one read and one write of the [rows, vocab] buffer instead of two reads and
    a write), and the backward scales the two products that consume that gradient by the upstream gradient of the
    loss, read from the device by their epilogues."""

    @staticmethod
    def forward(ctx, x, w, targets, V):
        x2 = _c(x).reshape(-1, x.shape[-1])
        t = _c(targets.reshape(-1))
        logits = G.mm_nt(x2, w, max_ctas=_max_ctas)
        loss_rows, _ = K.xent_fused_(logits, t, 1.0 / logits.shape[0], V)
        ctx.save_for_backward(x2, w, logits)
        ctx.x_shape = x.shape
        return K.mean_f32(loss_rows)

    @staticmethod
    def backward(ctx, dloss):
        x2, w, dlogits = ctx.saved_tensors
        g = _c(dloss.float()).reshape(1)
        if w.requires_grad:
            G.mm_tn_accum(dlogits, x2, main_grad(w), max_ctas=_max_ctas, alpha_dev=g)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = G.mm_nn(dlogits, w, max_ctas=_max_ctas, alpha_dev=g).reshape(ctx.x_shape)
        if w.requires_grad:
            _ready(w)   # after the data-gradient product, the last reader of w
        return dx, None, None, None


def linear_cross_entropy(x, w, targets, num_classes: int | None = None):
    """Mean cross-entropy of ``x @ w^T`` against ``targets`` (``w`` may carry padded rows past ``num_classes``).
    On CUDA bf16 this never keeps logits and their gradient as two tensors; elsewhere it is linear + cross_entropy."""
    V = num_classes or w.shape[0]
    if _nat(x) and torch.is_grad_enabled() and (x.requires_grad or w.requires_grad):
        return _LinearCrossEntropy.apply(x, w, targets, V)
    return cross_entropy(linear(x, w), targets, V)


def cross_entropy(logits, targets, num_classes: int | None = None):
    """Mean CE of ``logits[..., :num_classes]`` (extra padded columns are ignored)."""
    V = num_classes or logits.shape[-1]
    if _nat(logits):
        return _CrossEntropy.apply(logits, targets, V)
    return TF.cross_entropy(logits[..., :V].reshape(-1, V).float(), targets.reshape(-1))


# --------------------------------------------------------------------------------------------- attention
class _ComposedAttention(torch.autograd.Function):
    """Causal MHA with materialised scores: three batched tcgen05 GEMM launches + a softmax kernel.
    Slower than the online-softmax kernel; kept as the numerics reference and fallback."""

    @staticmethod
    def forward(ctx, qkv, H, D, scale):
        qkv = _c(qkv)
        B, T = qkv.shape[0], qkv.shape[1]
        Cm = H * D
        ld = 3 * Cm
        S = torch.empty(B * H, T, T, dtype=torch.bfloat16, device=qkv.device)
        G.gemm(qkv, qkv, S, M=T, N=T, K=D, lda=ld, ldb=ld, ldc=T, batch=(H, B), a_strides=(D, T * ld),
               b_strides=(D, T * ld), c_strides=(T * T, H * T * T), b_offset=Cm)
        K.causal_softmax_fwd_(S, T, scale)
        o = torch.empty(B, T, Cm, dtype=torch.bfloat16, device=qkv.device)
        G.gemm(S, qkv, o, M=T, N=D, K=T, lda=T, ldb=ld, ldc=Cm, b_mn=True, batch=(H, B),
               a_strides=(T * T, H * T * T), b_strides=(D, T * ld), c_strides=(D, T * Cm), b_offset=2 * Cm)
        ctx.save_for_backward(qkv, S)
        ctx.dims = (B, T, H, D, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, P = ctx.saved_tensors
        B, T, H, D, scale = ctx.dims
        do = _c(do)
        Cm = H * D
        ld = 3 * Cm
        dqkv = torch.empty_like(qkv)
        dP = torch.empty_like(P)
        pstr = (T * T, H * T * T)
        # dP = dO V^T
        G.gemm(do, qkv, dP, M=T, N=T, K=D, lda=Cm, ldb=ld, ldc=T, batch=(H, B), a_strides=(D, T * Cm),
               b_strides=(D, T * ld), c_strides=pstr, b_offset=2 * Cm)
        # dV = P^T dO
        G.gemm(P, do, dqkv, M=T, N=D, K=T, lda=T, ldb=Cm, ldc=ld, a_mn=True, b_mn=True, batch=(H, B),
               a_strides=pstr, b_strides=(D, T * Cm), c_strides=(D, T * ld), c_offset=2 * Cm)
        K.causal_softmax_bwd_(dP, P, T, scale)
        # dQ = dS K
        G.gemm(dP, qkv, dqkv, M=T, N=D, K=T, lda=T, ldb=ld, ldc=ld, b_mn=True, batch=(H, B), a_strides=pstr,
               b_strides=(D, T * ld), c_strides=(D, T * ld), b_offset=Cm)
        # dK = dS^T Q
        G.gemm(dP, qkv, dqkv, M=T, N=D, K=T, lda=T, ldb=ld, ldc=ld, a_mn=True, b_mn=True, batch=(H, B),
               a_strides=pstr, b_strides=(D, T * ld), c_strides=(D, T * ld), c_offset=Cm)
        return dqkv, None, None, None


def _attention_cpu(qkv, H, D, scale):
    B, T = qkv.shape[:2]
    q, k, v = qkv.view(B, T, 3, H, D).permute(2, 0, 3, 1, 4)
    o = TF.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale)
    return o.transpose(1, 2).reshape(B, T, H * D)


_attention_impl = "auto"


def set_attention_impl(name: str) -> None:
    """'flash' (online-softmax tcgen05 kernel), 'composed' (GEMM + softmax), or 'auto'."""
    global _attention_impl
    assert name in ("auto", "flash", "composed")
    _attention_impl = name


def causal_attention(qkv, n_heads: int, head_dim: int, scale: float | None = None):
    """Causal self-attention over a packed ``[B, T, 3*H*D]`` QKV tensor -> ``[B, T, H*D]``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if not _nat(qkv):
        return _attention_cpu(qkv, n_heads, head_dim, scale)
    impl = _attention_impl
    if impl in ("auto", "flash"):
        from . import attention as A
        if A.flash_supported(qkv, n_heads, head_dim):
            return A.flash_attention_packed(qkv, n_heads, head_dim, scale)
        if impl == "flash":
            raise nat.NativeError("flash attention kernel does not support this shape")
    return _ComposedAttention.apply(qkv, n_heads, head_dim, scale)


# --------------------------------------------------------------------------------------------- misc
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        gate_up = _c(gate_up)
        ctx.save_for_backward(gate_up)
        return K.swiglu_fwd(gate_up)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        return K.swiglu_bwd(_c(dy), gu)


def swiglu(gate_up):
    """``silu(gate) * up`` for a fused ``[..., 2F]`` gate/up projection output."""
    if _nat(gate_up):
        return _SwiGLU.apply(gate_up)
    g, u = gate_up.chunk(2, dim=-1)
    return TF.silu(g) * u


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, n_rot_heads, D, theta):
        # x: [B, T, Htot, D] packed heads; the first n_rot_heads heads (q and k) are rotated
        x = _c(x).clone()
        B, T, Ht, _ = x.shape
        K.rope_(x, B, T, n_rot_heads, D, T * Ht * D, Ht * D, D, theta, False)
        ctx.dims = (n_rot_heads, D, theta)
        return x

    @staticmethod
    def backward(ctx, dy):
        n, D, theta = ctx.dims
        dy = _c(dy).clone()
        B, T, Ht, _ = dy.shape
        K.rope_(dy, B, T, n, D, T * Ht * D, Ht * D, D, theta, True)
        return dy, None, None, None


def _rope_cpu(x, n, D, theta):
    B, T, Ht, _ = x.shape
    half = D // 2
    freq = theta ** (-2.0 * torch.arange(half, dtype=torch.float32, device=x.device) / D)
    ang = torch.arange(T, dtype=torch.float32, device=x.device)[:, None] * freq[None]
    cs, sn = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    r = x[:, :, :n].float()
    a, c = r[..., :half], r[..., half:]
    rot = torch.cat([a * cs - c * sn, c * cs + a * sn], dim=-1).to(x.dtype)
    return torch.cat([rot, x[:, :, n:]], dim=2)


def rope(x, n_rot_heads: int, head_dim: int, theta: float = 10000.0):
    """Rotary position embedding (rotate-half pairing) on the first ``n_rot_heads`` heads of [B,T,H,D]."""
    if _nat(x):
        return _Rope.apply(x, n_rot_heads, head_dim, theta)
    return _rope_cpu(x, n_rot_heads, head_dim, theta)


# --------------------------------------------------------------------------------------------- activations / dropout / conv
class _Activation(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, act):
        x = _c(x)
        ctx.save_for_backward(x)
        ctx.act = act
        return K.act_fwd(x, act)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return K.act_bwd(_c(dy), x, ctx.act), None


def activation(x, name: str):
    """Stand-alone GELU (exact erf) / SiLU for modules that do not fuse the activation into a GEMM epilogue."""
    if _nat(x):
        return _Activation.apply(x, ACT[name])
    return TF.gelu(x) if name == "gelu" else TF.silu(x)


class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        ctx.args = (p, seed, offset)
        return K.dropout(_c(x), p, seed, offset)

    @staticmethod
    def backward(ctx, dy):
        p, seed, offset = ctx.args
        return K.dropout(_c(dy), p, seed, offset), None, None, None   # same (seed, offset) -> same mask


def dropout(x, p: float, seed: int = 0, offset: int = 0):
    """Inverted dropout.  The mask is a pure function of (seed, offset, element index): it is regenerated in
    the backward pass instead of being stored."""
    if _nat(x):
        return _Dropout.apply(x, p, seed, offset)
    g = torch.Generator(device=x.device).manual_seed(seed * 1000003 + offset)
    mask = (torch.rand(x.shape, generator=g, device=x.device) >= p).to(x.dtype)
    return x * mask / (1.0 - p)


def conv2d_im2col(x, w, b, stride, padding, dilation):
    """bf16 CUDA convolution lowered to unfold + the tcgen05 GEMM (the reference lowers conv to im2col +
    its SGEMM per batch and group: crates/incin-backends/src/cuda/backend.rs:1638-1645)."""
    N, Cin, H, W = x.shape
    O, _, KH, KW = w.shape
    if x.requires_grad or not x.is_cuda:
        cols = TF.unfold(x, (KH, KW), dilation=dilation, padding=padding, stride=stride)   # [N, Cin*KH*KW, L]
        L = cols.shape[-1]
        a = cols.transpose(1, 2).reshape(N * L, Cin * KH * KW).contiguous()
    else:   # no gradient flows into the input (first layer, inference): the native unfold writes the GEMM operand directly
        from .tensor_ops import im2col
        a = im2col(x, (KH, KW), tuple(stride), tuple(padding), tuple(dilation))
        L = a.shape[0] // N
    kdim = a.shape[1]
    wk = w.reshape(O, kdim)
    if kdim % 8:   # TMA needs 16-byte row strides: pad the reduction dimension with zeros
        pad = 8 - kdim % 8
        a = TF.pad(a, (0, pad))
        wk = TF.pad(wk, (0, pad))
    y = linear(a, wk.contiguous(), b)
    oh = (H + 2 * padding[0] - dilation[0] * (KH - 1) - 1) // stride[0] + 1
    return y.reshape(N, L, O).transpose(1, 2).reshape(N, O, oh, L // oh)


def _gqa_cpu(qkv, Hq, Hkv, D, scale):
    B, T, _ = qkv.shape
    x = qkv.view(B, T, Hq + 2 * Hkv, D)
    q = x[:, :, :Hq].transpose(1, 2)
    k = x[:, :, Hq:Hq + Hkv].transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    v = x[:, :, Hq + Hkv:].transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    o = TF.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale)
    return o.transpose(1, 2).reshape(B, T, Hq * D)


def gqa_attention(qkv, n_heads: int, n_kv_heads: int, head_dim: int, scale: float | None = None):
    """Causal grouped-query attention over a packed ``[B, T, (Hq + 2 Hkv) * D]`` projection (query heads first,
    then key heads, then value heads) -> ``[B, T, Hq * D]``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if _nat(qkv):
        from . import attention as A
        if A.flash_supported(qkv, n_heads, head_dim, n_kv_heads):
            return A.flash_attention_packed(qkv, n_heads, head_dim, scale, n_kv_heads)
        raise nat.NativeError("no attention kernel for this head configuration (head_dim must be 64 or 128)")
    return _gqa_cpu(qkv, n_heads, n_kv_heads, head_dim, scale)
