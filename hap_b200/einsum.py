"""The four ``torch.einsum`` contractions of the reference's MoE layers on the batched tensor-core GEMM.

The planner emits ``torch.einsum(code, a, b)`` nodes for exactly four codes (``hap.rs:2255-2260,
2266-2276``; model side ``models.py:356-364``):

    "bsd,bsec->becd"   dispatch : expert_inputs = x (x) dispatch_tensor
    "edh,becd->bech"   expert FFN 1 (per-expert weights w1[e, d, h])
    "ehd,bech->becd"   expert FFN 2 (per-expert weights w2[e, h, d])
    "becd,bsec->bsd"   combine  : output = expert_outputs (x) combine_tensor

:func:`einsum` has ``torch.einsum``'s call surface for these codes (bfloat16, CUDA) with autograd.
Every contraction - forward and backward - is one call of ``hapx_gemm_batched``; operands are passed
as strided views (an index is allowed to be the contiguous one on either side of the contraction),
so the only copies are the (b, e) <-> (e, b) re-orderings that give the expert GEMMs b*c rows.
The two expert contractions return a (b, e, c, .) VIEW of (e, b, c, .) memory; values are identical.
"""
from __future__ import annotations

import torch

from . import _native as N
from .comm import _on_device, _stream

CODES = ("bsd,bsec->becd", "edh,becd->bech", "ehd,bech->becd", "becd,bsec->bsd")


def _major(t: torch.Tensor, what: str):
    """(mn_major, ld) of a [..., R, K] view: K-major when the last stride is 1, MN-major when the
    second-to-last is."""
    r, k = t.stride(-2), t.stride(-1)
    if k == 1 and (t.shape[-2] == 1 or r >= t.shape[-1]):
        return False, r if t.shape[-2] > 1 else max(r, t.shape[-1])
    if r == 1 and (t.shape[-1] == 1 or k >= t.shape[-2]):
        return True, k if t.shape[-1] > 1 else max(k, t.shape[-2])
    raise ValueError(f"einsum: {what} has no unit stride in its last two dimensions (strides {t.stride()})")


def bmm_nt(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """out[bo, bi, m, n] = sum_k a[bo, bi, m, k] * b[bo, bi, n, k] for 4-D bf16 views with arbitrary
    (8-element aligned) strides; ``b`` may be expanded (stride 0) along ``bo``."""
    if a.dim() != 4 or b.dim() != 4 or a.shape[:2] != b.shape[:2] or a.shape[3] != b.shape[3]:
        raise ValueError(f"bmm_nt: incompatible shapes {tuple(a.shape)} and {tuple(b.shape)}")
    for t in (a, b):
        if not t.is_cuda:
            raise RuntimeError(f"einsum: hap_b200 has no CPU path; tensor is on {t.device}")
        if t.dtype != torch.bfloat16:
            raise TypeError(f"einsum: bfloat16 only, got {t.dtype}")
    bo, bi, m, k = a.shape
    n = b.shape[2]
    a_mn, lda = _major(a, "first operand")
    b_mn, ldb = _major(b, "second operand")
    for v, what in ((lda, "row pitch"), (ldb, "row pitch"), (a.stride(1) if bi > 1 else 0, "batch stride"),
                    (a.stride(0) if bo > 1 else 0, "batch stride"), (b.stride(1) if bi > 1 else 0, "batch stride"),
                    (b.stride(0) if bo > 1 else 0, "batch stride")):
        if v % 8:
            raise ValueError(f"einsum: operand {what} {v} is not a multiple of 8 elements")
    out = torch.empty((bo, bi, m, n), dtype=out_dtype, device=a.device)
    with _on_device(a.device):
        N.check(N.lib.hapx_gemm_batched(out.data_ptr(), a.data_ptr(), b.data_ptr(), N.BF16 if out_dtype == torch.bfloat16 else N.F32,
                                        int(a_mn), int(b_mn), m, n, k, lda, ldb, n, bi, bo,
                                        a.stride(1) if bi > 1 else 0, a.stride(0) if bo > 1 else 0,
                                        b.stride(1) if bi > 1 else 0, b.stride(0) if bo > 1 else 0,
                                        m * n, bi * m * n, _stream(a.device)))
    return out


def _T(t):
    return t.transpose(-1, -2)


def _expert_major(t: torch.Tensor) -> torch.Tensor:
    """(b, e, c, x) -> contiguous-in-memory (e, b*c, x); free when t is already a view of such memory."""
    b, e, c, x = t.shape
    return t.permute(1, 0, 2, 3).contiguous().view(e, b * c, x)


class _Dispatch(torch.autograd.Function):          # "bsd,bsec->becd"
    @staticmethod
    def forward(ctx, x, disp):
        b, s, d = x.shape
        e, c = disp.shape[2], disp.shape[3]
        x, disp = x.contiguous(), disp.contiguous()
        ctx.save_for_backward(x, disp)
        out = bmm_nt(_T(disp.view(b, 1, s, e * c)), _T(x.view(b, 1, s, d)))
        return out.view(b, e, c, d)

    @staticmethod
    def backward(ctx, g):
        x, disp = ctx.saved_tensors
        b, s, d = x.shape
        e, c = disp.shape[2], disp.shape[3]
        g2 = g.contiguous().view(b, 1, e * c, d)
        dx = ddisp = None
        if ctx.needs_input_grad[0]:
            dx = bmm_nt(disp.view(b, 1, s, e * c), _T(g2)).view(b, s, d)
        if ctx.needs_input_grad[1]:
            ddisp = bmm_nt(x.view(b, 1, s, d), g2).view(b, s, e, c)
        return dx, ddisp


class _ExpertLinear(torch.autograd.Function):      # "edh,becd->bech" and "ehd,bech->becd"
    @staticmethod
    def forward(ctx, w, inp):
        e, kin, kout = w.shape
        b, _, c, _ = inp.shape
        w = w.contiguous()
        ie = _expert_major(inp)                                       # (e, b*c, kin)
        ctx.save_for_backward(w, ie)
        ctx.bc = (b, c)
        out = bmm_nt(ie.view(1, e, b * c, kin), _T(w).unsqueeze(0))  # B(n = kout, k = kin) = w[e, kin, kout]^T
        return out.view(e, b, c, kout).permute(1, 0, 2, 3)

    @staticmethod
    def backward(ctx, g):
        w, ie = ctx.saved_tensors
        e, kin, kout = w.shape
        b, c = ctx.bc
        ge = _expert_major(g)                                         # (e, b*c, kout)
        dw = dinp = None
        if ctx.needs_input_grad[0]:
            dw = bmm_nt(_T(ie).unsqueeze(0), _T(ge).unsqueeze(0)).view(e, kin, kout)
        if ctx.needs_input_grad[1]:
            dinp = bmm_nt(ge.view(1, e, b * c, kout), w.unsqueeze(0)).view(e, b, c, kin).permute(1, 0, 2, 3)
        return dw, dinp


class _Combine(torch.autograd.Function):           # "becd,bsec->bsd"
    @staticmethod
    def forward(ctx, eo, comb):
        b, e, c, d = eo.shape
        s = comb.shape[1]
        eo, comb = eo.contiguous(), comb.contiguous()
        ctx.save_for_backward(eo, comb)
        out = bmm_nt(comb.view(b, 1, s, e * c), _T(eo.view(b, 1, e * c, d)))
        return out.view(b, s, d)

    @staticmethod
    def backward(ctx, g):
        eo, comb = ctx.saved_tensors
        b, e, c, d = eo.shape
        s = comb.shape[1]
        g2 = g.contiguous().view(b, 1, s, d)
        deo = dcomb = None
        if ctx.needs_input_grad[0]:
            deo = bmm_nt(_T(comb.view(b, 1, s, e * c)), _T(g2)).view(b, e, c, d)
        if ctx.needs_input_grad[1]:
            dcomb = bmm_nt(g2, eo.view(b, 1, e * c, d)).view(b, s, e, c)
        return deo, dcomb


# ---- sparse dispatch / combine ---------------------------------------------------------------------
# The dispatch and combine tensors of a gating function hold at most one token per (expert, capacity)
# slot and at most two slots per token (models.py:477-502), so the two einsums that use them are row
# gathers.  :func:`sparse_dispatch` / :func:`sparse_combine` compute the same values as
# ``einsum("bsd,bsec->becd", x, dispatch)`` / ``einsum("becd,bsec->bsd", expert_out, combine)`` for such
# tensors; :func:`hap_b200.fxpass.sparsify_moe` puts them in place of the einsum nodes whose second
# operand comes straight out of a gating function.
def _moe_index(dense: torch.Tensor):
    b, s, e, c = dense.shape
    dense = dense.contiguous()
    dev = dense.device
    slot_token = torch.empty((b, e * c), dtype=torch.int32, device=dev)
    slot_weight = torch.empty((b, e * c), dtype=torch.float32, device=dev)
    token_slot = torch.empty((b, s, 2), dtype=torch.int32, device=dev)
    token_weight = torch.empty((b, s, 2), dtype=torch.float32, device=dev)
    with _on_device(dev):
        N.check(N.lib.hapx_moe_index(dense.data_ptr(), slot_token.data_ptr(), slot_weight.data_ptr(), token_slot.data_ptr(),
                                     token_weight.data_ptr(), b, s, e * c, _stream(dev)))
    return slot_token, slot_weight, token_slot, token_weight


def _token_view(t: torch.Tensor) -> torch.Tensor:
    """A (b, s, d) token tensor the kernels can address in place: rows contiguous, both strides multiples of 8
    elements (any dense permutation of (b, s) qualifies, e.g. a view of sequence-major memory); a copy otherwise."""
    if t.stride(2) == 1 and t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


def _rows_view(rows: torch.Tensor):
    """(tensor, capacity flag) for a (b, e, c, d) row tensor: 0 for batch-major memory, c for expert-major memory
    (a permuted view of a contiguous (e, b, c, d) tensor - what the expert GEMMs produce); a copy otherwise."""
    if rows.is_contiguous():
        return rows, 0
    if rows.permute(1, 0, 2, 3).is_contiguous():
        return rows, rows.shape[2]
    return rows.contiguous(), 0


def _new_rows(b, e, c, d, like: torch.Tensor, expert_major: bool) -> torch.Tensor:
    if expert_major:
        return torch.empty((e, b, c, d), dtype=like.dtype, device=like.device).permute(1, 0, 2, 3)
    return torch.empty((b, e, c, d), dtype=like.dtype, device=like.device)


def _rows_from_tokens(x, slot_token, slot_weight, e, c, expert_major=False):
    b, s, d = x.shape
    x = _token_view(x)
    rows = _new_rows(b, e, c, d, x, expert_major)
    with _on_device(x.device):
        N.check(N.lib.hapx_moe_rows_from_tokens_strided(rows.data_ptr(), x.data_ptr(), slot_token.data_ptr(),
                                                        slot_weight.data_ptr() if slot_weight is not None else None, b, s, e * c, d,
                                                        x.stride(0), x.stride(1), c if expert_major else 0, _stream(x.device)))
    return rows


def _tokens_from_rows(rows, token_slot, token_weight, s, sequence_major=False):
    """rows: (b, e, c, d) in either memory layout; the (b, s, d) result is a view of sequence-major memory when
    asked (so that a gradient comes out in the layout of the tensor it belongs to)."""
    b, e, c, d = rows.shape
    rows, cap = _rows_view(rows)
    if sequence_major:
        y = torch.empty((s, b, d), dtype=rows.dtype, device=rows.device).permute(1, 0, 2)
    else:
        y = torch.empty((b, s, d), dtype=rows.dtype, device=rows.device)
    with _on_device(rows.device):
        N.check(N.lib.hapx_moe_tokens_from_rows_strided(y.data_ptr(), rows.data_ptr(), token_slot.data_ptr(),
                                                        token_weight.data_ptr() if token_weight is not None else None, b, s, e * c, d,
                                                        y.stride(0), y.stride(1), cap, _stream(rows.device)))
    return y


def _check_sparse(a: torch.Tensor, dense: torch.Tensor, what: str) -> None:
    for t in (a, dense):
        if not t.is_cuda:
            raise RuntimeError(f"{what}: hap_b200 has no CPU path; tensor is on {t.device}")
        if t.dtype != torch.bfloat16:
            raise TypeError(f"{what}: bfloat16 only, got {t.dtype}")
    if a.shape[-1] % 8:
        raise ValueError(f"{what}: the model dimension must be a multiple of 8")


class _SparseDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, disp, expert_major):
        b, s, e, c = disp.shape
        slot_token, slot_weight, token_slot, token_weight = _moe_index(disp)
        ctx.save_for_backward(token_slot, token_weight)
        ctx.meta = (s, e, c)
        ctx.x_sequence_major = (not x.is_contiguous()) and x.permute(1, 0, 2).is_contiguous()
        return _rows_from_tokens(x, slot_token, slot_weight, e, c, expert_major)

    @staticmethod
    def backward(ctx, g):
        token_slot, token_weight = ctx.saved_tensors
        s, e, c = ctx.meta
        if ctx.needs_input_grad[1]:
            raise NotImplementedError("sparse_dispatch: the dispatch tensor is a constant of the gating function ((combine > 0), models.py:500)")
        dx = None
        if ctx.needs_input_grad[0]:
            dx = _tokens_from_rows(g, token_slot, token_weight, s, ctx.x_sequence_major)
        return dx, None, None


class _SparseCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, eo, comb, sequence_major):
        b, e, c, d = eo.shape
        s = comb.shape[1]
        slot_token, slot_weight, token_slot, token_weight = _moe_index(comb)
        eo, cap = _rows_view(eo)
        ctx.save_for_backward(eo, slot_token, slot_weight, token_slot)
        ctx.meta = (s, e, c, cap)
        return _tokens_from_rows(eo, token_slot, token_weight, s, sequence_major)

    @staticmethod
    def backward(ctx, g):
        eo, slot_token, slot_weight, token_slot = ctx.saved_tensors
        s, e, c, cap = ctx.meta
        b, d = eo.shape[0], eo.shape[3]
        g = _token_view(g)
        deo = dcomb = None
        if ctx.needs_input_grad[0]:
            deo = _rows_from_tokens(g, slot_token, slot_weight, e, c, expert_major=cap != 0)     # in the layout of the rows it belongs to
        if ctx.needs_input_grad[1]:
            dcomb = torch.empty((b, s, e, c), dtype=g.dtype, device=g.device)
            with _on_device(g.device):
                N.check(N.lib.hapx_moe_weight_grad_strided(dcomb.data_ptr(), eo.data_ptr(), g.data_ptr(), token_slot.data_ptr(), b, s, e * c, d,
                                                           g.stride(0), g.stride(1), cap, _stream(g.device)))
        return deo, dcomb, None


def sparse_dispatch(x: torch.Tensor, dispatch: torch.Tensor, expert_major: bool = False) -> torch.Tensor:
    """``einsum("bsd,bsec->becd", x, dispatch)`` for a gating function's dispatch tensor, as a row gather.
    ``expert_major``: return the (b, e, c, d) result as a view of (e, b, c, d) memory, the layout the expert GEMMs
    read - for when they consume it directly (no all_to_all in between)."""
    _check_sparse(x, dispatch, "sparse_dispatch")
    return _SparseDispatch.apply(x, dispatch, bool(expert_major))


def sparse_combine(expert_out: torch.Tensor, combine: torch.Tensor, sequence_major: bool = False) -> torch.Tensor:
    """``einsum("becd,bsec->bsd", expert_out, combine)`` for a gating function's combine tensor, as a weighted
    gather of at most two rows per token.  The gradient w.r.t. ``combine`` is produced at the positions
    where ``combine`` is non-zero - the only ones a gating function's backward reads.  ``sequence_major``: return
    the (b, s, d) result as a view of (s, b, d) memory - for a program that transposes it right away."""
    _check_sparse(expert_out, combine, "sparse_combine")
    return _SparseCombine.apply(expert_out, combine, bool(sequence_major))


def einsum(code: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``torch.einsum(code, a, b)`` for the four MoE contractions of the reference."""
    code = code.replace(" ", "")
    if code == "bsd,bsec->becd":
        return _Dispatch.apply(a, b)
    if code in ("edh,becd->bech", "ehd,bech->becd"):
        return _ExpertLinear.apply(a, b)
    if code == "becd,bsec->bsd":
        return _Combine.apply(a, b)
    raise NotImplementedError(f"einsum: the planner only emits {CODES}; got {code!r}")
