"""Grouped (per-expert) SwiGLU MLP over rows sorted by expert: the reference's three ``hnn.MoELinear`` ragged dots
(src/levanter/models/mixtral.py:245-277).

Rows ``[sum(group_sizes), hidden]`` are contiguous per expert.  Each expert's slice runs through the tcgen05 GEMM
(gate and up projections, the gated-activation kernel, then the down projection); expert boundaries are read back once
per call."""
from __future__ import annotations

import torch

from ..utils.activation import ActivationFunctionEnum
from .gemm import linear
from .glu import gated_activation


def grouped_mlp(x_sorted: torch.Tensor, group_sizes: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor,
                act: ActivationFunctionEnum, first_expert: int = 0) -> torch.Tensor:
    """``out[rows of expert e] = (act(x w1[e]^T) * (x w3[e]^T)) w2[e]^T``; ``w1/w3: [E, mlp, hidden]``, ``w2: [E, hidden, mlp]``.
    ``group_sizes`` covers the experts held in ``w*`` starting at global expert ``first_expert``."""
    sizes = group_sizes.tolist()
    n_local = w1.shape[0]
    sizes = sizes[first_expert:first_expert + n_local] if len(sizes) != n_local else sizes
    outs = []
    start = 0
    dt = x_sorted.dtype
    for e, n in enumerate(sizes):
        if n == 0:
            continue
        xe = x_sorted[start:start + n]
        a, b, c = w1[e], w3[e], w2[e]
        if a.dtype != dt:
            a, b, c = a.to(dt), b.to(dt), c.to(dt)
        h = gated_activation(linear(xe, a), linear(xe, b), act)
        outs.append(linear(h, c))
        start += n
    if not outs:
        return x_sorted.new_zeros((0, w2.shape[1]))
    return torch.cat(outs, dim=0)


# ------------------------------------------------------------------------------------------------ padded grouped path
# Rows sorted by expert with every expert's segment padded to a multiple of 128 rows: no row block of the GEMM kernel
# straddles two experts, the expert boundaries stay on the device (no host read-back, so the step can be captured in a
# CUDA graph), and one launch covers all experts (``lvb_gemm_grouped``).
BLOCK = 128


def padded_layout(expert_of_row: torch.Tensor, num_experts: int):
    """For ``expert_of_row[R]`` (the expert each (token, choice) pair goes to) returns, all on the device:
    ``dest[R]``: row of every pair in the padded sorted buffer; ``offsets[E + 1]``: padded start row of every expert;
    ``tile_group[capacity / 128]``: expert of every 128-row block (-1 past the end); and the static ``capacity``."""
    R = expert_of_row.numel()
    E = num_experts
    capacity = ((R + E * (BLOCK - 1)) + BLOCK - 1) // BLOCK * BLOCK
    idx = expert_of_row.reshape(-1).long()
    counts = torch.bincount(idx, minlength=E)
    padded = (counts + BLOCK - 1) // BLOCK * BLOCK
    offsets = torch.zeros(E + 1, dtype=torch.long, device=idx.device)
    offsets[1:] = torch.cumsum(padded, 0)
    starts = torch.zeros(E, dtype=torch.long, device=idx.device)
    starts[1:] = torch.cumsum(counts, 0)[:-1]
    order = torch.argsort(idx, stable=True)
    rank_sorted = torch.empty_like(order)
    rank_sorted[order] = torch.arange(R, device=idx.device)
    dest = offsets[idx] + (rank_sorted - starts[idx])
    blocks = torch.arange(capacity // BLOCK, device=idx.device)
    tile_group = torch.searchsorted(offsets[1:] // BLOCK, blocks, right=True)
    tile_group = torch.where(blocks < offsets[E] // BLOCK, tile_group, torch.full_like(tile_group, -1))
    return dest, offsets.to(torch.int32), tile_group.to(torch.int32), capacity


def _grouped_fn():
    from . import lib

    c = lib
    return lib.fn("lvb_gemm_grouped", [c.c_int, c.c_void_p, c.c_void_p, c.c_void_p] + [c.c_int] * 9 + [c.c_float, c.c_void_p, c.c_void_p,
                                                                                                     c.c_void_p, c.c_void_p])


_g = {}


def _grouped(kind, a, b, out, groups, Tp, M, N, K, flags, tile_group, offsets):
    from . import lib

    if "f" not in _g:
        _g["f"] = _grouped_fn()
    rc = _g["f"](kind, a.data_ptr(), b.data_ptr(), out.data_ptr(), groups, Tp, M, N, K, a.stride(0), b.stride(-2), out.stride(-2), flags, 1.0,
                 lib.ptr(tile_group), lib.ptr(offsets), lib.status_buffer().data_ptr(), lib.stream_ptr())
    lib.check_rc(rc, "lvb_gemm_grouped")
    return out


def _use_grouped_kernel(x: torch.Tensor, w: torch.Tensor) -> bool:
    from . import lib

    return x.is_cuda and lib.available() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % BLOCK == 0 \
        and w.shape[2] % 8 == 0


class _GroupedLinear(torch.autograd.Function):
    """``y[rows of expert e] = x[rows of e] w[e]^T`` over the padded layout; ``w``: ``[E, out, in]``."""

    @staticmethod
    def forward(ctx, x, w, tile_group, offsets):
        E, N, K = w.shape
        Tp = x.shape[0]
        y = torch.empty(Tp, N, dtype=x.dtype, device=x.device)
        _grouped(0, x, w, y, E, Tp, 0, N, K, 0, tile_group, None)
        ctx.save_for_backward(x, w, tile_group, offsets)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, tile_group, offsets = ctx.saved_tensors
        E, N, K = w.shape
        Tp = x.shape[0]
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(Tp, K, dtype=x.dtype, device=x.device)
            _grouped(1, dy, w, dx, E, Tp, 0, K, N, 0, tile_group, None)
            # row blocks past the last expert were skipped by the kernel: their gradient is zero, not whatever the buffer held
            dx = torch.where((tile_group >= 0).repeat_interleave(BLOCK).unsqueeze(1), dx, torch.zeros((), dtype=dx.dtype, device=dx.device))
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            if main is not None:
                _grouped(2, dy, x, main, E, Tp, N, K, 0, 1 | 2, None, offsets)  # fp32, accumulate into the engine's buffer
                dw = None
            else:
                acc = torch.zeros(E, N, K, dtype=torch.float32, device=x.device)
                _grouped(2, dy, x, acc, E, Tp, N, K, 0, 1 | 2, None, offsets)
                dw = acc.to(w.dtype)
        return dx, dw, None, None


def grouped_linear(x_pad: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    if _use_grouped_kernel(x_pad, w):
        return _GroupedLinear.apply(x_pad, w, tile_group, offsets)
    # reference: one matmul per expert over its padded segment (CPU path and test oracle)
    off = offsets.tolist()
    y = x_pad.new_zeros(x_pad.shape[0], w.shape[1])
    for e in range(w.shape[0]):
        if off[e + 1] > off[e]:
            y[off[e]:off[e + 1]] = x_pad[off[e]:off[e + 1]] @ w[e].to(x_pad.dtype).t()
    return y


def grouped_mlp_padded(x_flat: torch.Tensor, topk_idx: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor,
                       act: ActivationFunctionEnum) -> torch.Tensor:
    """Expert MLP of every (token, choice) pair: ``x_flat[T, hidden]``, ``topk_idx[T, k]`` -> ``[T * k, hidden]`` in pair order.
    Permutation into the padded layout, three grouped GEMMs with the gated activation in between, permutation back."""
    T, k = topk_idx.shape
    E = w1.shape[0]
    dest, offsets, tile_group, capacity = padded_layout(topk_idx.reshape(-1), E)
    x_pad = x_flat.new_zeros(capacity, x_flat.shape[1])
    x_pad = x_pad.index_copy(0, dest, x_flat.repeat_interleave(k, dim=0))
    dt = x_flat.dtype
    if w1.dtype != dt:
        w1, w3, w2 = w1.to(dt), w3.to(dt), w2.to(dt)
    h = gated_activation(grouped_linear(x_pad, w1, tile_group, offsets), grouped_linear(x_pad, w3, tile_group, offsets), act)
    y = grouped_linear(h, w2, tile_group, offsets)
    return y.index_select(0, dest)


def grouped_mlp_on_padded(x_pad: torch.Tensor, tile_group: torch.Tensor, offsets: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor,
                          w2: torch.Tensor, act: ActivationFunctionEnum) -> torch.Tensor:
    """The expert MLP over rows that are already in the padded expert-sorted layout (``offsets[E + 1]`` padded starts,
    ``tile_group`` the expert of every 128-row block, both on the device): what the expert-parallel exchange delivers."""
    dt = x_pad.dtype
    if w1.dtype != dt:
        w1, w3, w2 = w1.to(dt), w3.to(dt), w2.to(dt)
    h = gated_activation(grouped_linear(x_pad, w1, tile_group, offsets), grouped_linear(x_pad, w3, tile_group, offsets), act)
    return grouped_linear(h, w2, tile_group, offsets)


# ------------------------------------------------------------------------------------------------ routing
def moe_route_reference(router_logits: torch.Tensor, k: int):
    """``(topk_w[T, k], topk_idx[T, k], counts[E], p_sum[E], lse[T])`` with PyTorch ops (CPU path and oracle)."""
    z = router_logits.float()
    probs = torch.softmax(z, dim=-1)
    w, idx = torch.topk(probs, k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    counts = torch.bincount(idx.reshape(-1), minlength=z.shape[-1])
    return w, idx, counts, probs.sum(0), torch.logsumexp(z, dim=-1)


class _MoeRoute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k):
        from . import lib

        c = lib
        T, E = logits.shape
        z = logits.float().contiguous()
        dev = z.device
        idx = torch.empty(T, k, dtype=torch.int32, device=dev)
        w = torch.empty(T, k, dtype=torch.float32, device=dev)
        probs = torch.empty(T, E, dtype=torch.float32, device=dev)
        lse = torch.empty(T, dtype=torch.float32, device=dev)
        counts = torch.zeros(E, dtype=torch.int32, device=dev)
        psum = torch.empty(E, dtype=torch.float32, device=dev)
        scratch = torch.empty(((T + 127) // 128) * E, dtype=torch.float32, device=dev)
        f = lib.fn("lvb_moe_route_fwd", [c.c_void_p, c.c_int, c.c_int, c.c_int] + [c.c_void_p] * 8, launches=2)
        rc = f(z.data_ptr(), T, E, k, idx.data_ptr(), w.data_ptr(), probs.data_ptr(), lse.data_ptr(), counts.data_ptr(), psum.data_ptr(),
               scratch.data_ptr(), lib.stream_ptr())
        lib.check_rc(rc, "lvb_moe_route_fwd")
        ctx.save_for_backward(probs, idx)
        ctx.k = k
        ctx.in_dtype = logits.dtype
        idx64 = idx.long()
        ctx.mark_non_differentiable(idx64, counts)
        return w, idx64, counts, psum, lse

    @staticmethod
    def backward(ctx, d_w, _d_idx, _d_counts, d_psum, d_lse):
        from . import lib

        c = lib
        probs, idx = ctx.saved_tensors
        T, E = probs.shape
        dz = torch.empty_like(probs)
        prep = lambda t: None if t is None else t.float().contiguous()  # noqa: E731
        d_w, d_psum, d_lse = prep(d_w), prep(d_psum), prep(d_lse)
        f = lib.fn("lvb_moe_route_bwd", [c.c_void_p] * 5 + [c.c_int] * 3 + [c.c_void_p, c.c_void_p])
        rc = f(probs.data_ptr(), idx.data_ptr(), lib.ptr(d_w), lib.ptr(d_psum), lib.ptr(d_lse), T, E, ctx.k, dz.data_ptr(), lib.stream_ptr())
        lib.check_rc(rc, "lvb_moe_route_bwd")
        return dz.to(ctx.in_dtype), None


def moe_route(router_logits: torch.Tensor, k: int):
    """Routing of ``router_logits[T, E]``: renormalised top-``k`` weights and indices, tokens per expert, per-expert sums of
    the router probabilities (for the load-balancing loss) and the per-token log-sum-exp (for the router z-loss).
    Differentiable in the weights, the probability sums and the log-sum-exp."""
    from . import lib

    E = router_logits.shape[-1]
    if router_logits.is_cuda and lib.available() and E <= 64 and k <= 8:
        return _MoeRoute.apply(router_logits, k)
    return moe_route_reference(router_logits, k)
