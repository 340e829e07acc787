"""The kernel library as the parts see it: one method per kernel, tensors in, nothing
out (outputs are arguments).  The methods check what the kernels cannot check for
themselves and pass raw device pointers to the ``extern "C"`` launchers of the
shared library built from ``csrc/``.

The reference reaches its kernels through a name-keyed callback table
("<op>_<CPU|GPU>_<dtype>", src/kernel/include/TFFOPCreatorBase.h:62-101) with a CPU
twin for some ops.  There is one backend here: sm_100a.  If the library cannot be
built or loaded, or a tensor is not on a CUDA device, the call fails loudly; nothing
falls back to another implementation.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import numpy as np
import torch

from ..csrc import build as _build

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_vp = ctypes.c_void_p

_STATUS = {
    -1: "bad argument (a size or pointer the kernel cannot take)",
    -2: "unsupported size for this kernel",
    -3: "kernel launch failed",
    -4: "CUDA driver entry point unavailable",
    -5: "a bounded wait inside a kernel ran out",
}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return _vp(t.data_ptr()) if t is not None else _vp(0)


def effective_requests(kv_lens) -> float:
    """sum(context) / max(context): how many requests of the longest context read as many keys as these
    do.  A step's decoded tokens are one (request, key/value head) work item each unless the key range is
    shared out; the longest context sets how long the longest item runs, the sum how long all of them
    take together, so this ratio, not the number of requests, says how many shares the key range needs."""
    kv = np.asarray(kv_lens, dtype=np.float64)
    if kv.size == 0 or kv.max() <= 0:
        return 1.0
    return float(kv.sum() / kv.max())


def nearest_power_of_two(x: float) -> int:
    b = 1
    while b * 1.4142 < x:
        b *= 2
    return b


class DeferredNorm:
    """A norm that has not been run yet: the float32 rows ``x``, the weight and eps of an RMSNorm whose
    output only feeds a product of the kernel library.  ``CudaKernels.gated_mlp`` takes it in place of the
    activation rows and runs norm, product and SwiGLU as one kernel when the shape allows (decode steps of at
    most 16 tokens in bfloat16: csrc/gemm_tc_cluster.cu); otherwise, and in ``qkv_project``, the norm kernel
    runs first (``materialize``)."""
    def __init__(self, x, weight, eps, out_dtype, ops):
        self.x, self.weight, self.eps, self.out_dtype, self.ops = x, weight, float(eps), out_dtype, ops
        self.shape = x.shape
        self.dtype = out_dtype
        self.device = x.device

    def materialize(self):
        out = torch.empty(self.x.shape, dtype=self.out_dtype, device=self.x.device)
        self.ops.rmsnorm(self.x, self.weight, self.eps, out)
        return out


class CudaKernels:
    """Loads (building first if needed) the sm_100a kernel library."""

    def __init__(self, verbose_build: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("tffinfer_b200 needs a CUDA device (sm_100a): torch.cuda.is_available() is False")
        path = _build.library_path(build=True, verbose=verbose_build)
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        self.path = path
        self.launches = 0          # number of kernel launches issued through this object
        self._accumulators = {}    # (shape, device) -> float32 buffer kept at zero between uses
        self._acc_zero = {}        # data_ptr -> True while the buffer is known to hold zeros
        self._inv_freq_cache = {}
        # the planners below cut work by the SM count the launchers size their grids with
        self.NUM_SMS = int(self.lib.tff_sm_count())
        if self.NUM_SMS <= 0:
            raise KernelError("cannot read the SM count of the current CUDA device")

    # ------------------------------------------------------------- plumbing
    @staticmethod
    def _stream():
        return _vp(torch.cuda.current_stream().cuda_stream)

    def _check(self, status: int, what: str) -> None:
        if status != 0:
            raise KernelError(f"{what}: {_STATUS.get(status, f'status {status}')}")

    @staticmethod
    def _need_cuda(*tensors) -> None:
        for t in tensors:
            if t is not None and not t.is_cuda:
                raise KernelError("a tensor given to a CUDA kernel is not on a CUDA device")
            if t is not None and not t.is_contiguous():
                raise KernelError("kernels take contiguous tensors")

    @staticmethod
    def _cache_args(kv_cache, kv_layer: int):
        """(pointer, pages, layers, layer) of a paged cache [pages, layers, 2, kv heads, page, head] as the
        launchers take them.  The tensor is either contiguous as it reads (pages outermost), or that shape
        as a view of storage with the layers outermost, each layer's pages then lying together (what the
        engine allocates: a layer's attention reads addresses within one layer's share of the pool and not
        64 KB out of every ``layers`` x 64 KB).  For the second the launcher is given the layer's own
        [pages, 1, ...] block."""
        if kv_cache is None:
            return _vp(0), 0, 1, kv_layer
        if not kv_cache.is_cuda:
            raise KernelError("a tensor given to a CUDA kernel is not on a CUDA device")
        if kv_cache.is_contiguous():
            return _vp(kv_cache.data_ptr()), kv_cache.shape[0], kv_cache.shape[1], kv_layer
        st, block = kv_cache.stride(), 1
        for i in range(kv_cache.dim() - 1, 1, -1):             # the [2, kv heads, page, head] block of a page is dense
            if st[i] != block:
                break
            block *= kv_cache.shape[i]
        else:
            if st[0] == block and st[1] == block * kv_cache.shape[0]:
                return (_vp(kv_cache.data_ptr() + kv_layer * st[1] * kv_cache.element_size()),
                        kv_cache.shape[0], 1, 0)
        raise KernelError("the cache is neither contiguous nor a view of layer-major storage")

    # -------------------------------------------------------------- kernels
    def embed(self, token_ids, table, out, scale: float = 1.0) -> None:
        self._need_cuda(token_ids, table, out)
        T, H = out.shape
        assert token_ids.dtype == torch.int32 and out.dtype == torch.float32 and table.shape[1] == H
        self._check(self.lib.tff_embed(_ptr(token_ids), _ptr(table), _c_int(_dt(table)), _ptr(out),
                                       _c_int(T), _c_int(H), _c_int(table.shape[0]), _c_float(scale), self._stream()), "embed")
        self.launches += 1

    def logit_transform(self, logits, scale: float = 1.0, softcap: float = 0.0) -> None:
        """In place: logits * scale, then softcap * tanh(. / softcap) when softcap > 0."""
        self._need_cuda(logits)
        assert logits.dtype == torch.float32
        self._check(self.lib.tff_logit_transform(_ptr(logits), ctypes.c_longlong(logits.numel()), _c_float(scale),
                                                 _c_float(softcap), self._stream()), "logit_transform")
        self.launches += 1

    def rmsnorm(self, x, weight, eps: float, out, row_index=None) -> None:
        self._need_cuda(x, weight, out, row_index)
        rows, dim = out.shape
        assert x.dtype == torch.float32 and weight.dtype == torch.float32 and x.shape[1] == dim
        assert weight.numel() == dim
        if row_index is not None:
            assert row_index.dtype == torch.int32 and row_index.numel() == rows
        else:
            assert x.shape[0] == rows
        self._check(self.lib.tff_rmsnorm(_ptr(x), _ptr(weight), _ptr(row_index), _ptr(out), _c_int(_dt(out)),
                                         _c_int(rows), _c_int(dim), _c_float(eps), self._stream()), "rmsnorm")
        self.launches += 1

    def gemm(self, a, w, out, residual=None) -> None:
        """out[M, N] = a[M, K] @ w[N, K]^T (+ residual, float32 [M, N]; may be ``out``)."""
        self._need_cuda(a, w, out, residual)
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K and tuple(out.shape) == (M, N)
        if residual is not None:
            assert residual.dtype == torch.float32 and tuple(residual.shape) == (M, N)
            assert out.dtype == torch.float32
        self._gemm_dispatch(a, w, out, residual, M, N, K)

    def _gemm_dispatch(self, a, w, out, residual, M, N, K) -> None:
        if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            self.gemm_tc(a, w, out, residual)
        else:
            self.gemm_simt(a, w, out, residual)

    def gemm_simt(self, a, w, out, residual=None) -> None:
        """Plain-FMA float32-accumulate product for any mix of float32 / bfloat16 operands."""
        M, K = a.shape
        N = w.shape[0]
        self._check(self.lib.tff_gemm_simt(_ptr(a), _c_int(_dt(a)), _ptr(w), _c_int(_dt(w)), _ptr(out),
                                           _c_int(_dt(out)), _ptr(residual), _c_int(M), _c_int(N), _c_int(K),
                                           self._stream()), "gemm_simt")
        self.launches += 1

    FOLD_MAX_M = 16           # up to this many rows the norm is folded into the gate/up product (with SwiGLU)
    CLUSTER_MAX_M = 16        # up to this many rows the gate/up product applies SwiGLU itself (clusters share a tile's K range)
    FOLD_DECODE = os.environ.get("TFFINFER_FOLD_DECODE", "1") != "0"
    SWAP_MAX_M = 256          # up to this many rows the weights are the 128-row operand
    USE_SM_PAIRS = os.environ.get("TFFINFER_SM_PAIRS", "1") != "0"   # prompt-sized products on tcgen05 cta_group::2
    NUM_SMS = 0               # SMs of the device, read from it when the library is loaded

    def tc_plan(self, M: int, N: int, K: int, out_is_f32: bool, add: bool = False):
        """(swap, bn, stream_k) of the tcgen05 product for a shape.  stream_k: 0 = whole tiles; 1 = the
        (tile, K block) units in equal contiguous shares; S >= 2 = the tiles of the last, partial wave
        in S slices of their K range."""
        if M <= self.SWAP_MAX_M:
            bn = 16
            while bn < M:
                bn *= 2
            tiles = -(-N // 128)
            stream_k = 1 if (out_is_f32 and tiles < 4 * self.NUM_SMS) else 0
            return 1, bn, stream_k
        return self.prompt_plan(M, N, K, add and out_is_f32)

    # What a wave of tiles costs in each of the three prompt-sized configurations, in us per K block of 64 at the
    # clocks of a B200 under load, and what a launch costs on top: fitted to the measured times of the q/k/v, o,
    # gate/up and down products of the 8B and 14B shapes at 160 to 544 rows (within 10 %; only the ratios matter).
    # A tile of the last wave costs as much as one of a full wave, so the plan with the fewest waves wins unless
    # its tiles are the dearer ones: 544 rows of the 14B shape's q/k/v are 84 pair tiles on 74 pairs of SMs (two
    # waves, 63 us) and 140 single tiles on 148 SMs (one wave, 38 us).
    #          bn: (us a K block and wave, us a launch, tile rows, tile columns, SMs a tile)
    TILE_COST = {512: (0.385, 3.0, 256, 256, 2), 256: (0.450, 1.0, 128, 256, 1), 128: (0.340, 1.5, 128, 128, 1)}

    def prompt_costs(self, M: int, N: int, K: int, added: bool, kinds=(512, 256, 128)):
        """{bn: (estimated us, slices)} of the normal-orientation configurations for a prompt-sized product; the
        last wave's tiles are cut along K only where the result is added to a float32 buffer."""
        kb = -(-K // 64)
        costs = {}
        for bn in kinds:
            if bn == 512 and (not self.USE_SM_PAIRS or N <= 128):
                continue
            c, launch, tm, tn, sms = self.TILE_COST[bn]
            tiles, slots = -(-M // tm) * -(-N // tn), max(1, self.NUM_SMS // sms)
            waves, tail = divmod(tiles, slots)
            slices = self.tail_slices(tiles, kb, slots) if added else 0
            if tail:
                waves += (-(-tail * slices // slots) / slices + 0.02 * slices) if slices else 1
            costs[bn] = (waves * kb * c + launch, slices)
        return costs

    def prompt_plan(self, M: int, N: int, K: int, added: bool, kinds=(512, 256, 128)):
        """(0, bn, slices) of the cheapest of them."""
        costs = self.prompt_costs(M, N, K, added, kinds)
        bn = min(costs, key=lambda b: costs[b][0])
        return 0, bn, costs[bn][1]

    @staticmethod
    def tail_slices(tiles: int, k_blocks: int, ctas: int) -> int:
        """In how many slices the K range of the tiles of the last wave is cut (0: not at all).  A wave of
        R tiles in S slices takes ceil(R*S/G)/S of a tile's time; every slice costs another pass of the
        tile through the epilogue, here put at 2 % of a tile's time."""
        tail = tiles % ctas
        if tail == 0:
            return 0
        best, best_cost = 0, 1.0
        for s in range(2, min(8, k_blocks) + 1):
            cost = -(-tail * s // ctas) / s + 0.02 * s
            if cost < best_cost - 1e-9:
                best, best_cost = s, cost
        return best

    def gemm_tc(self, a, w, out, residual=None, plan=None) -> None:
        """bfloat16 x bfloat16 product on the tensor cores (tcgen05), float32 accumulation."""
        M, K = a.shape
        N = w.shape[0]
        swap, bn, stream_k = plan if plan is not None else self.tc_plan(M, N, K, out.dtype == torch.float32,
                                                                        residual is not None)
        add = 0
        if residual is not None:
            assert out.dtype == torch.float32
            if residual.data_ptr() != out.data_ptr():
                out.copy_(residual)
            add = 1
        elif stream_k:
            assert out.dtype == torch.float32
            if not self._acc_zero.get(out.data_ptr(), False):
                self.zero_f32(out)            # shares of a split tile are added to it
        if out.data_ptr() in self._acc_zero:
            self._acc_zero[out.data_ptr()] = False
        self._check(self.lib.tff_gemm_tc(_ptr(a), _ptr(w), _ptr(out), _c_int(_dt(out)), _c_int(add),
                                         _c_int(M), _c_int(N), _c_int(K), _c_int(swap), _c_int(bn), _c_int(stream_k),
                                         self._stream()), "gemm_tc")
        self.launches += 1

    def zero_f32(self, t) -> None:
        assert t.dtype == torch.float32 and t.is_contiguous()
        self._check(self.lib.tff_zero_f32(_ptr(t), ctypes.c_longlong(t.numel()), self._stream()), "zero_f32")
        self.launches += 1

    def reset_state_slots(self, state, slots, pos_start) -> None:
        """state[slots[b]] = 0 for every request b of the step whose first token is at position 0.
        state: [slots, ...] of any element type; slots, pos_start: int32 [B] on the device."""
        self._need_cuda(state, slots, pos_start)
        assert slots.dtype == pos_start.dtype == torch.int32 and slots.numel() == pos_start.numel()
        slot_bytes = state[0].numel() * state.element_size()
        self._check(self.lib.tff_reset_state_slots(_ptr(state), ctypes.c_longlong(slot_bytes), _c_int(state.shape[0]),
                                                   _ptr(slots), _ptr(pos_start), _c_int(slots.numel()),
                                                   self._stream()), "reset_state_slots")
        self.launches += 1

    def gather_tokens(self, token_ids, drawn, src) -> None:
        """token_ids[i] = drawn[src[i]] wherever src[i] >= 0 (all int32, on the device)."""
        self._need_cuda(token_ids, drawn, src)
        assert token_ids.dtype == drawn.dtype == src.dtype == torch.int32 and src.numel() == token_ids.numel()
        self._check(self.lib.tff_gather_tokens(_ptr(token_ids), _ptr(drawn), _ptr(src), _c_int(token_ids.numel()),
                                               _c_int(drawn.numel()), self._stream()), "gather_tokens")
        self.launches += 1

    def error_word_async(self, pinned: torch.Tensor, index: int) -> None:
        """Copies the kernels' error word into element ``index`` of a pinned int32 host tensor, in stream
        order; non-zero there (once the stream has got that far) means check_errors() will raise."""
        assert pinned.dtype == torch.int32 and pinned.is_pinned() and 0 <= index < pinned.numel()
        self._check(self.lib.tff_error_word_to_host_async(_vp(pinned.data_ptr() + 4 * index), self._stream()),
                    "error_word_to_host")

    def selftest_bounded_wait(self, arrive: bool, max_polls: int = 4096) -> None:
        """Launches a kernel that waits, bounded, on a barrier at which one thread arrives (``arrive``) or
        nobody does: in the second case the wait runs out after ``max_polls`` polls and raises the error
        word, as a stalled pipeline inside a tcgen05 kernel would.  For testing the way from the word to
        the caller (error_word_async, check_errors)."""
        self._check(self.lib.tff_selftest_bounded_wait(_c_int(1 if arrive else 0), _c_int(max_polls), self._stream()),
                    "selftest_bounded_wait")
        self.launches += 1

    def check_errors(self) -> None:
        """Synchronises and raises if a bounded wait inside a kernel ran out since the last check."""
        v = self.lib.tff_kernel_error()
        if v != 0:
            raise KernelError("a bounded wait inside a tcgen05 kernel ran out (or the error word could not be read)")

    @staticmethod
    def gate_up_block(inter: int) -> int:
        """Layout of a merged gate/up weight: 64 = gate and up rows alternate in blocks of 64 (what the
        fused tensor-core epilogue wants), 0 = all gate rows, then all up rows."""
        return 64 if inter % 64 == 0 else 0

    def merge_gate_up(self, gate_w, up_w):
        """One weight [2I, K] from the gate and up projections, in the layout gemm_swiglu expects."""
        I, K = gate_w.shape
        b = self.gate_up_block(I)
        if b == 0:
            return torch.cat([gate_w, up_w], dim=0).contiguous()
        return torch.stack([gate_w.view(I // b, b, K), up_w.view(I // b, b, K)], dim=1).reshape(2 * I, K).contiguous()

    # ------------------------------------------------------- accumulator buffers
    def projection_buffer(self, rows: int, width: int, device, act_dtype) -> torch.Tensor:
        """A float32 [rows, width] buffer for a projection's accumulators.  For decode-sized bfloat16
        batches it is a persistent buffer that is zero now and that its reader sets back to zero
        (``release_input`` of qk_norm_rope_kv_write, ``clear`` of swiglu), so that the split product
        can add into it without a clearing kernel; otherwise it is plain scratch."""
        if act_dtype != torch.bfloat16 or rows > self.SWAP_MAX_M:
            return torch.empty((rows, width), dtype=torch.float32, device=device)
        key = (rows, width, str(device))
        buf = self._accumulators.get(key)
        if buf is None:
            buf = torch.zeros((rows, width), dtype=torch.float32, device=device)
            self._accumulators[key] = buf
            self._acc_zero[buf.data_ptr()] = True
        return buf

    def reset_accumulators(self) -> None:
        """After a step that was cut short: every accumulator buffer back to zero."""
        for buf in self._accumulators.values():
            buf.zero_()
            self._acc_zero[buf.data_ptr()] = True

    # ------------------------------------------------------- folded decode products
    def can_fold_norm(self, x, weight, out_dtype) -> bool:
        """Whether an RMSNorm of these rows may be handed to the products as a DeferredNorm."""
        return (self.FOLD_DECODE and x.is_cuda and out_dtype == torch.bfloat16 and x.dtype == torch.float32
                and x.dim() == 2 and x.shape[0] <= self.FOLD_MAX_M and x.shape[1] % 8 == 0 and x.is_contiguous()
                and weight.dtype == torch.float32 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)

    def _foldable_weight(self, w) -> bool:
        return w.dtype == torch.bfloat16 and w.is_contiguous() and w.data_ptr() % 16 == 0 and w.shape[1] % 8 == 0

    def gated_mlp(self, h, w_gate_up, w_down, residual, inter: int) -> None:
        """residual += down(silu(gate(h)) * up(h)); ``h`` the activation rows or a DeferredNorm of them.
        A decode step of at most FOLD_MAX_M tokens in bfloat16 whose norm has been deferred runs two kernels:
        norm, gate/up product and SwiGLU as one (clusters of CTAs share a tile's K range), then the down
        product.  Everything else runs the products and kernels one by one."""
        T = h.shape[0]
        if isinstance(h, DeferredNorm):
            if (self.gate_up_block(inter) == 64 and self._foldable_weight(w_gate_up)
                    and residual.is_cuda and residual.dtype == torch.float32):
                act = torch.empty((T, inter), dtype=torch.bfloat16, device=residual.device)
                self._need_cuda(h.x, h.weight, w_gate_up, act)
                assert tuple(w_gate_up.shape) == (2 * inter, h.x.shape[1])
                self._check(self.lib.tff_gemm_tc_cluster_swiglu(
                    _ptr(h.x), _ptr(h.weight), _c_float(h.eps), _ptr(w_gate_up), _c_int(T), _c_int(h.x.shape[1]),
                    _ptr(act), _c_int(inter), self._stream()), "gemm_tc_cluster_swiglu")
                self.launches += 1
                self.gemm(act, w_down, residual, residual=residual)
                return
            h = h.materialize()
        act = torch.empty((T, inter), dtype=h.dtype, device=h.device)
        if (self.FOLD_DECODE and T <= self.CLUSTER_MAX_M and h.dtype == torch.bfloat16 and h.is_cuda and h.is_contiguous()
                and self.gate_up_block(inter) == 64 and self._foldable_weight(w_gate_up) and h.data_ptr() % 16 == 0):
            # the product with SwiGLU in the first CTA of each cluster: no float32 accumulators, no SwiGLU kernel
            self._need_cuda(h, w_gate_up, act)
            assert tuple(w_gate_up.shape) == (2 * inter, h.shape[1])
            self._check(self.lib.tff_gemm_tc_cluster_swiglu_bf16(_ptr(h), _ptr(w_gate_up), _c_int(T), _c_int(h.shape[1]),
                                                                 _ptr(act), _c_int(inter), self._stream()),
                        "gemm_tc_cluster_swiglu_bf16")
            self.launches += 1
        else:
            self.gemm_swiglu(h, w_gate_up, act)
        self.gemm(act, w_down, residual, residual=residual)

    def swiglu(self, gate_up, out, block: int = 0) -> None:
        """out[t, i] = silu(gate[t, i]) * up[t, i]; gate_up float32 or of out's type, [gate | up] (block = 0) or
        alternating in blocks of ``block`` columns."""
        self._need_cuda(gate_up, out)
        T, I = out.shape
        assert gate_up.shape == (T, 2 * I) and gate_up.dtype in (torch.float32, out.dtype)
        clear = 1 if gate_up.data_ptr() in self._acc_zero else 0
        self._check(self.lib.tff_swiglu(_ptr(gate_up), _c_int(_dt(gate_up)), _ptr(out), _c_int(_dt(out)),
                                        _c_int(T), _c_int(I), _c_int(block), _c_int(clear), self._stream()), "swiglu")
        if clear:
            self._acc_zero[gate_up.data_ptr()] = True
        self.launches += 1

    def rope_table(self, table, theta: float, rot_dim: int) -> None:
        """table float32 [max_pos, rot_dim/2, 2] = (cos, sin)(pos * theta^(-2i/rot_dim)).
        The frequencies exp(-(2i/d) ln theta) (src/kernel/cuda/rope_table.cu:33) are
        evaluated in double on the host and rounded once to float32."""
        self._need_cuda(table)
        half = rot_dim // 2
        assert table.dtype == torch.float32 and tuple(table.shape[1:]) == (half, 2)
        i = np.arange(half, dtype=np.float64)
        inv = np.exp(-(2.0 * i / float(rot_dim)) * math.log(theta)).astype(np.float32)
        inv_t = torch.from_numpy(inv).to(table.device)
        self._check(self.lib.tff_rope_table(_ptr(table), _ptr(inv_t), _c_int(table.shape[0]), _c_int(rot_dim),
                                            self._stream()), "rope_table")
        torch.cuda.current_stream().synchronize()   # inv_t must outlive the kernel
        self.launches += 1

    def qk_norm_rope_kv_write(self, qkv, q_out, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache,
                              kv_layer, page_size, nq, nkv, d, write_cache) -> None:
        """qkv [T, (nq+2nkv)*d] float32 or activation type -> q_out [T, nq*d] (normed, rotated) and the
        token's K/V page slots."""
        self._need_cuda(qkv, q_out, q_w, k_w, table, block_table)
        c_ptr, _, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        T = qkv.shape[0]
        assert qkv.shape[1] == (nq + 2 * nkv) * d and tuple(q_out.shape) == (T, nq * d)
        assert qkv.dtype in (torch.float32, q_out.dtype)
        if write_cache:
            assert kv_cache is not None and kv_cache.dtype == q_out.dtype, "cache dtype must match activations"
            assert tuple(kv_cache.shape[2:]) == (2, nkv, page_size, d)
        clear = 1 if qkv.data_ptr() in self._acc_zero else 0
        self._check(self.lib.tff_qk_norm_rope_kv_write(
            _ptr(qkv), _c_int(1 if qkv.dtype == torch.float32 else 0), _c_int(clear), _ptr(q_out), _c_int(_dt(q_out)),
            _ptr(q_w), _ptr(k_w), _c_float(eps),
            _ptr(table), _c_int(rot_dim), _c_int(table.shape[0] if table is not None else 0),
            _ptr(batch.positions), _ptr(batch.tok_req), _ptr(block_table),
            _c_int(block_table.shape[1] if block_table is not None else 0),
            c_ptr, _c_int(c_layers), _c_int(c_layer), _c_int(page_size), _c_int(1 if write_cache else 0),
            _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d), self._stream()), "qk_norm_rope_kv_write")
        if clear:
            self._acc_zero[qkv.data_ptr()] = True
        self.launches += 1

    def qkv_project(self, h, w_qkv, q_out, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache,
                    kv_layer, page_size, nq, nkv, d, write_cache) -> None:
        """The q/k/v projection of ``h`` with ``w_qkv`` ([q heads | k heads | v heads] rows), per-head RMSNorm of
        q and k, rotation, q into ``q_out`` and k, v into the tokens' cache slots.  The projection's accumulators
        stay in float32 until q and k have been normalised.  Prompt-sized bfloat16 batches with heads of 128 do all
        of it in the epilogue of the product on pairs of SMs; everything else is the product into a float32 buffer
        followed by qk_norm_rope_kv_write."""
        T, K = h.shape
        if isinstance(h, DeferredNorm):
            h = h.materialize()
        # The fused form runs on pairs of SMs only.  Where another configuration saves more waves than the separate
        # kernel costs (a pass over the float32 projection at about 5 TB/s and a launch), the projection is not fused.
        if self.USE_SM_PAIRS and T > self.SWAP_MAX_M:
            costs = self.prompt_costs(T, (nq + 2 * nkv) * d, K, False)
            apart = min(v[0] for v in costs.values()) + T * (nq + 2 * nkv) * d * 6 / 5e6 + 3.0
            pairs_pay = 512 in costs and costs[512][0] <= apart
        else:
            pairs_pay = False
        fused = (pairs_pay and d == 128 and h.dtype == torch.bfloat16
                 and w_qkv.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16 and K % 8 == 0
                 and (table is None or rot_dim == d) and (kv_cache is None or kv_cache.dtype == torch.bfloat16)
                 and (not write_cache or kv_cache is not None)
                 and all(t is None or t.data_ptr() % 16 == 0 for t in (h, w_qkv, q_out, q_w, k_w, table, kv_cache))
                 and (kv_cache is None or kv_cache.stride(0) % 8 == 0 and kv_cache.stride(1) % 8 == 0))
        if not fused:
            qkv = self.projection_buffer(T, (nq + 2 * nkv) * d, h.device, h.dtype)
            self.gemm(h, w_qkv, qkv)
            self.qk_norm_rope_kv_write(qkv, q_out, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache,
                                       kv_layer, page_size, nq, nkv, d, write_cache)
            return
        self._need_cuda(h, w_qkv, q_out, q_w, k_w, table, block_table)
        c_ptr, _, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        assert tuple(w_qkv.shape) == ((nq + 2 * nkv) * d, K) and tuple(q_out.shape) == (T, nq * d)
        if write_cache:
            assert tuple(kv_cache.shape[2:]) == (2, nkv, page_size, d)
        self._check(self.lib.tff_gemm_tc_qkv_rope(
            _ptr(h), _ptr(w_qkv), _c_int(T), _c_int(K), _ptr(q_out), _ptr(q_w), _ptr(k_w), _c_float(eps),
            _ptr(table), _c_int(table.shape[0] if table is not None else 0),
            _ptr(batch.positions), _ptr(batch.tok_req), _ptr(block_table),
            _c_int(block_table.shape[1] if block_table is not None else 0),
            c_ptr, _c_int(c_layers), _c_int(c_layer), _c_int(page_size), _c_int(1 if write_cache else 0),
            _c_int(nq), _c_int(nkv), self._stream()), "gemm_tc_qkv_rope")
        self.launches += 1

    def attend(self, h, w_qkv, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache, kv_layer, page_size, out,
               nq, nkv, d, scale, window, write_cache) -> None:
        """The whole mixer between its input rows and its output projection: q/k/v projection of ``h``, per-head
        RMSNorm of q and k, rotation, cache write, attention over the paged cache -> out [T, nq*d].  How many
        kernels that is, is decided here: prompt portions with heads of 128 do everything up to the cache write in
        the projection's epilogue (qkv_project); a decode step runs projection, q/k-norm + rotation + write, and
        attention (with the merge of its key shares).  A decode attention that took the projection's float32
        accumulators and finished queries, new keys and new values itself was built and measured: one launch
        fewer and 0.05 ms a step slower at the Qwen3-8B shape (under programmatic dependent launch the small
        kernel's time already hid behind the attention's first loads of old keys), so it was not kept."""
        T = h.shape[0]
        q = torch.empty((T, nq * d), dtype=out.dtype, device=out.device)
        self.qkv_project(h, w_qkv, q, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache, kv_layer, page_size,
                         nq, nkv, d, write_cache)
        self.attention(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale, window)

    def attention(self, q, batch, block_table, kv_cache, kv_layer, page_size, out,
                  nq, nkv, d, scale, window) -> None:
        """q [T, nq*d] (normed, rotated) against the paged cache -> out [T, nq*d]."""
        self._need_cuda(q, block_table, out)
        T = q.shape[0]
        assert kv_cache.dtype == q.dtype == out.dtype
        assert tuple(q.shape) == (T, nq * d) and tuple(out.shape) == (T, nq * d)
        assert tuple(kv_cache.shape[2:]) == (2, nkv, page_size, d)
        self._attention_dispatch(q, batch, block_table, kv_cache, kv_layer, page_size, out,
                                 nq, nkv, d, scale, window)

    def _attention_dispatch(self, q, batch, block_table, kv_cache, kv_layer, page_size, out,
                            nq, nkv, d, scale, window) -> None:
        if q.dtype == torch.bfloat16 and d in (64, 128):
            self.attention_bf16(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale, window)
        else:
            self.attention_generic(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale, window)

    def attention_splits(self, num_requests: float, max_q_len: int, nq: int, nkv: int) -> int:
        """Shares of the key range per tile, for ``num_requests`` requests of one context length (for
        unequal contexts: sum / longest, effective_requests above).  The count is rounded to a
        power of two, so that a step replayed as a CUDA graph, captured for such a class, and an eager
        step cut alike."""
        if max_q_len * (nq // nkv) > 16:
            return 1                                   # portions: enough tiles already
        b = nearest_power_of_two(num_requests)
        # One wave of two CTAs per SM.  With more work items than that the grid runs in rounds and the last one is
        # seldom full (64 requests of 8 heads on 296 slots: two rounds for 1.73 rounds' worth of work); cutting
        # the items so that the rounds fill was measured and lost (4 shares: 7.36 against 6.76 ms a step at 64
        # requests): every share pays its own ramp, and the partial results another pass.
        return max(1, min(16, 2 * self.NUM_SMS // (b * nkv)))

    MIXED_SHARES_FROM = 6144      # keys behind a small portion from which it is cut into shares beside decoded tokens too

    def portion_splits(self, num_requests: int, max_q_len: int, max_kv_len: int, nq: int, nkv: int) -> int:
        """Shares of the key range for a step that is prompt portions only.  A portion of few tokens behind a long
        context (the last piece of a prompt, what a step's token budget left over) is one or two tiles a key/value
        head: as tensor-core tiles of 128 rows they walk the whole context on 8 or 16 SMs.  Up to 256 packed rows
        (tokens times query heads a key/value head) behind 2,048 keys or more, such portions go to the kernel of
        64-row tiles with the key range cut into shares, as many as give every SM two CTAs.  A whole step of the
        8B shape with 16 tokens behind 4,000: 7.2 -> 5.1 ms; behind 16,000: 16.1 -> 6.8; 64 behind 16,000: 14.5 ->
        10.1; behind 1,000 keys it loses (5.4 -> 5.6), and above 256 rows the tensor-core kernel is the faster one
        (96 tokens behind 2,048: 60 against 65 us a layer)."""
        rows = max_q_len * (nq // nkv)
        if rows <= 16 or rows > 256 or max_kv_len < 2048:
            return 1
        ctas = -(-rows // 64) * nkv * max(1, num_requests)
        blocks = -(-max_kv_len // 64)
        s = 1
        while s < 16 and ctas * s * 2 <= 2 * self.NUM_SMS and s * 2 <= blocks:
            s *= 2
        return s

    @staticmethod
    def key_split_class(kv_lens) -> int:
        """The class of a batch of decoded tokens that fixes how their key ranges are shared out: a step
        replayed as a CUDA graph is captured per class."""
        return nearest_power_of_two(effective_requests(kv_lens))

    def _side_stream(self, device):
        """The second stream (and the two events to fork to it and join from it), made at first use."""
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=device)
            self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()
        return self._side

    def _decode_splits(self, batch, first: int, count: int, max_q_len: int, nq: int, nkv: int) -> int:
        """The key split for requests [first, first + count) in the order of ``batch.req_order``."""
        if batch.key_split_class is not None:
            eff = batch.key_split_class
        elif batch.h_sorted_kv_lens is not None:
            eff = effective_requests(batch.h_sorted_kv_lens[first:first + count])
        else:
            eff = count
        return self.attention_splits(eff, max_q_len, nq, nkv)

    def attention_bf16(self, q, batch, block_table, kv_cache, kv_layer, page_size, out,
                       nq, nkv, d, scale, window, num_splits=None) -> None:
        """Flash attention over the paged cache (head sizes 64 and 128).  Requests that bring so few
        tokens that they fit a 16-row tile (decoded tokens) and requests that bring long portions are
        launched apart when a step holds both, each with the kernel made for it."""
        G = nq // nkv
        sq = batch.h_sorted_q_lens
        B = batch.num_requests
        n_short = int(np.searchsorted(sq, 16 // G, side="right")) if (sq is not None and num_splits is None) else 0
        if 0 < n_short < B and batch.req_order is not None:
            # The two launches write different rows of ``out`` and read what the kernels before them wrote:
            # they run side by side, the decoded tokens' on a second stream.  The portions' kernel is
            # launched first; it seldom fills the SMs (a 512-token portion is 80 to 160 CTAs of one an SM),
            # and the other one, bound by memory, runs on what is left.
            main = torch.cuda.current_stream()
            side = None if torch.cuda.is_current_stream_capturing() else self._side_stream(q.device)
            if side is not None:
                self._fork.record(main)
            # (One share for the portions here unless their context is long: their few CTAs run beside the decoded
            # tokens' kernel, which has the other SMs; cut into shares they contend with it for all of them.  Measured:
            # the 14B mixed workload, contexts up to 4,096, 3.52-3.61 s with shares against 3.35-3.37 without; a step of
            # the 8B shape with 16 tokens behind 4,000 keys beside 8 decoded tokens 8.2 against 8.1 ms, behind 8,000 keys
            # 8.1 against 10.6, behind 16,000 keys 8.1 against 15.9.)
            long_kv = int(batch.h_sorted_kv_lens[n_short:].max()) if batch.h_sorted_kv_lens is not None else 0
            shares = self.portion_splits(B - n_short, int(sq[-1]), long_kv, nq, nkv) if long_kv >= self.MIXED_SHARES_FROM else 1
            self._attention_bf16_launch(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale,
                                        window, shares, batch.req_order[n_short:], B - n_short, int(sq[-1]))
            splits = self._decode_splits(batch, 0, n_short, int(sq[n_short - 1]), nq, nkv)
            if side is None:
                self._attention_bf16_launch(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d,
                                            scale, window, splits, batch.req_order[:n_short], n_short,
                                            int(sq[n_short - 1]))
            else:
                side.wait_event(self._fork)
                with torch.cuda.stream(side):
                    self._attention_bf16_launch(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv,
                                                d, scale, window, splits, batch.req_order[:n_short], n_short,
                                                int(sq[n_short - 1]))
                    self._join.record(side)
                main.wait_event(self._join)
        else:
            if num_splits is None:
                if batch.max_q_len * G > 16:
                    num_splits = self.portion_splits(B, batch.max_q_len, batch.max_kv_len, nq, nkv)
                else:
                    num_splits = self._decode_splits(batch, 0, B, batch.max_q_len, nq, nkv)
            # decoded tokens only: longest contexts first (the order the batch was packed with)
            order = batch.req_order if n_short == B else None
            self._attention_bf16_launch(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale,
                                        window, num_splits, order, B, batch.max_q_len)

    def _attention_bf16_launch(self, q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale,
                               window, num_splits, req_ids, num_requests, max_q_len) -> None:
        T = q.shape[0]
        splits = num_splits
        c_ptr, c_pages, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        ws = None
        if splits > 1:
            need = T * nq * splits * (d + 2)
            if max_q_len * (nq // nkv) > 16:
                # portions cut into shares: one buffer that only grows, since their sizes change from step to step and
                # a fresh size may cost an allocation from the driver in the middle of serving
                ws = getattr(self, "_portion_ws", None)
                if ws is None or ws.numel() < need or ws.device != q.device:
                    ws = torch.empty(max(need, 1 << 22), dtype=torch.float32, device=q.device)
                    self._portion_ws = ws
            else:
                ws = torch.empty(need, dtype=torch.float32, device=q.device)
        self._check(self.lib.tff_attention_bf16_paged(
            _ptr(q), _ptr(batch.q_start), _ptr(batch.pos_start), _ptr(req_ids), _ptr(block_table),
            _c_int(block_table.shape[1]),
            c_ptr, ctypes.c_longlong(c_pages), _c_int(c_layers), _c_int(c_layer),
            _c_int(page_size),
            _ptr(out), _ptr(ws), _c_int(T), _c_int(num_requests), _c_int(max_q_len), _c_int(splits),
            _c_int(nq), _c_int(nkv), _c_int(d), _c_float(scale), _c_int(window), self._stream()), "attention_bf16")
        self.launches += 2 if splits > 1 else 1

    def attention_generic(self, q, batch, block_table, kv_cache, kv_layer, page_size, out,
                          nq, nkv, d, scale, window) -> None:
        T = q.shape[0]
        c_ptr, _, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        self._check(self.lib.tff_attention_generic(
            _ptr(q), _c_int(_dt(q)), _c_int(q.shape[1]),
            _ptr(batch.positions), _ptr(batch.tok_req), _ptr(block_table), _c_int(block_table.shape[1]),
            c_ptr, _c_int(c_layers), _c_int(c_layer), _c_int(page_size),
            _ptr(out), _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d), _c_float(scale), _c_int(window),
            self._stream()), "attention_generic")
        self.launches += 1

    def gemm_swiglu(self, a, w_gate_up, out) -> None:
        """out[T, I] = silu(a @ Wg^T) * (a @ Wu^T), w_gate_up being merge_gate_up(Wg, Wu)."""
        self._need_cuda(a, w_gate_up, out)
        T, I = out.shape
        K = a.shape[1]
        block = self.gate_up_block(I)
        tc = (a.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and K % 8 == 0
              and a.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0)
        if tc and T > self.CLUSTER_MAX_M and block == 64 and out.dtype == torch.bfloat16 and out.data_ptr() % 16 == 0:
            # the activation is applied in the product's epilogue, in the normal orientation from 17 rows on: the
            # swapped product and the SwiGLU kernel behind it took 45 us at 72 rows of the 8B shape against 39, 78
            # against 59 at 256
            bn = self.prompt_plan(T, 2 * I, K, False)[1]
            self._check(self.lib.tff_gemm_tc_swiglu(_ptr(a), _ptr(w_gate_up), _ptr(out), _c_int(T), _c_int(I),
                                                    _c_int(K), _c_int(bn), self._stream()),
                        "gemm_tc_swiglu")
            self.launches += 1
            return
        small = tc and T <= self.SWAP_MAX_M
        if small:
            gu = self.projection_buffer(T, 2 * I, out.device, out.dtype)
        else:
            gu = torch.empty((T, 2 * I), dtype=out.dtype, device=out.device)
        self.gemm(a, w_gate_up, gu)
        self.swiglu(gu, out, block)
    def argmax(self, logits, out) -> None:
        self._need_cuda(logits, out)
        R, V = logits.shape
        assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() == R
        scratch = getattr(self, "_argmax_scratch", None)
        if scratch is None or scratch.device != logits.device:
            # 64 ticket counters (kept at zero by the kernel), then the candidates of 16 shares for up to 64 rows
            scratch = torch.zeros(64 + 2 * 64 * 16, dtype=torch.int32, device=logits.device)
            self._argmax_scratch = scratch
        use = scratch
        self._check(self.lib.tff_argmax(_ptr(logits), _ptr(out), _c_int(R), _c_int(V), _ptr(use), self._stream()), "argmax")
        self.launches += 1

    def sample(self, logits, temperature, uniform, out, top_k=None, top_p=None, min_p=None) -> None:
        self._need_cuda(logits, temperature, uniform, out, top_k, top_p, min_p)
        R, V = logits.shape
        assert logits.dtype == torch.float32 and out.dtype == torch.int32
        assert temperature.dtype == torch.float32 and uniform.dtype == torch.float32
        self._check(self.lib.tff_sample(_ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(top_k), _ptr(top_p),
                                        _ptr(min_p), _ptr(out), _c_int(R), _c_int(V), self._stream()), "sample")
        self.launches += 1

    def repetition_penalty(self, logits, rows, tokens, penalty) -> None:
        self._need_cuda(logits, rows, tokens, penalty)
        n = rows.numel()
        assert logits.dtype == torch.float32 and rows.dtype == torch.int32 and tokens.dtype == torch.int32
        assert penalty.dtype == torch.float32 and tokens.numel() == n and penalty.numel() == n
        self._check(self.lib.tff_repetition_penalty(_ptr(logits), _ptr(rows), _ptr(tokens), _ptr(penalty),
                                                    _c_int(n), _c_int(logits.shape[1]), self._stream()),
                    "repetition_penalty")
        self.launches += 1
