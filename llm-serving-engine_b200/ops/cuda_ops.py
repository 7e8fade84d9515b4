"""The kernel set of the product path: thin, checked calls into the sm_100a extension.

There is no other implementation behind these methods: if CUDA or the compiled extension is not
available, constructing :class:`CudaOps` raises.

Matrix products: float32 runs this package's own CUDA-core kernel (true 32-bit, no tensor-core
mode). bfloat16 products go to cuBLAS through ``torch.mm`` with float32 accumulation, the same
library-for-linear-layers split as the reference (src/llmserve/models/layers.py:129-152).
"""

from __future__ import annotations

import numpy as np
import torch

from . import build

_DTYPES = (torch.float32, torch.bfloat16)


class CudaOps:
    name = "cuda-sm100a"

    def __init__(self, device: torch.device | str = "cuda") -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise RuntimeError(
                "llmserve_b200 runs on a CUDA device only (built for sm_100a); no CPU fallback exists"
            )
        self.ext = build.load_core()
        self._attn_loaded: set[int] = set()
        self._scratch: torch.Tensor | None = None
        self._sample_scratch: torch.Tensor | None = None
        self._sample_rows = 0
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.attention_kernel = 0  # 0: fastest available; 1: CUDA cores; 2: mma.sync (tests compare them)
        self.use_skinny_gemm = True
        self.skinny_max_rows = int(self.ext.gemm_bf16_skinny_max_rows())
        self.skinny_atomic_rows = 32  # measured: above this the library's kernels are faster
        # float32 accumulation buffers of the few-rows product, by shape. Invariant: a buffer that
        # is not in _ws_live reads as zero (the kernel that consumes a product zeroes what it reads).
        self._addmm_in_place: bool | None = None  # whether torch.addmm can add into a float32 tensor
        self._ws: dict[tuple[int, int], torch.Tensor] = {}
        self._ws_live: dict[int, tuple[int, int]] = {}  # data_ptr -> shape of products not yet consumed
        self.launches = 0  # kernels of this package enqueued (library matrix products not counted)

    # ------------------------------------------------------------------ capabilities
    def branch_dtype(self, dtype: torch.dtype) -> torch.dtype:
        """Dtype in which projections that feed the residual stream return their result."""
        return torch.float32

    def check_attention_shape(self, head_dim: int, dtype: torch.dtype) -> None:
        if dtype not in _DTYPES:
            raise ValueError(f"attention kernels exist for float32 and bfloat16, not {dtype}")
        if head_dim not in self._attn_loaded:
            self.ext.load_attention_library(build.attention_library(head_dim), head_dim)
            self._attn_loaded.add(head_dim)

    def reserve_attention_scratch(self, head_dim: int, max_decode: int, num_heads: int,
                                  max_splits: int = 64) -> None:
        """Allocate the partial-result buffer of split-context attention once, at its largest."""
        need = int(self.ext.attention_scratch_floats(head_dim, max_decode, num_heads, max_splits))
        if self._scratch is None or self._scratch.numel() < need:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("attention scratch must be reserved before graph capture")
            # zeros: the buffer starts with completion counters that every launch leaves at zero
            self._scratch = torch.zeros(need, dtype=torch.float32, device=self.device)

    def check_kernel_errors(self) -> None:
        """Raise if a kernel recorded that one of its bounded waits ran out."""
        code = int(self.ext.kernel_error())
        if code:
            self.ext.clear_kernel_error()
            raise RuntimeError(f"a CUDA kernel of llmserve_b200 gave up waiting (code {code})")

    # ------------------------------------------------------------------ pointwise
    def embedding(self, token_ids, table):
        out = torch.empty(token_ids.shape[0], table.shape[1], dtype=torch.float32, device=table.device)
        self.ext.embedding(token_ids, table, out)
        self.launches += 1
        return out

    def add_rmsnorm(self, x, residual, weight, eps, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device)
        self.ext.add_rmsnorm(x, residual, weight, float(eps), out, rows)
        self.launches += 1
        return out

    def _accumulator(self, T: int, N: int) -> torch.Tensor:
        """A zero float32 ``[T, N]`` buffer for atomic sums: the persistent one of this shape if its
        last product has been consumed, else a fresh one."""
        ws = self._ws.get((T, N))
        if ws is None and not torch.cuda.is_current_stream_capturing():
            ws = self._ws[(T, N)] = torch.zeros(T, N, dtype=torch.float32, device=self.device)
        if ws is None or ws.data_ptr() in self._ws_live:
            return torch.zeros(T, N, dtype=torch.float32, device=self.device)
        self._ws_live[ws.data_ptr()] = (T, N)
        return ws

    def _consumes(self, t: torch.Tensor, out_dtype, kernel_can_zero: bool) -> bool:
        """True if ``t`` is a live accumulation buffer that the consuming kernel will zero."""
        if t.data_ptr() not in self._ws_live:
            return False
        if t.dtype == torch.float32 and out_dtype == torch.bfloat16 and kernel_can_zero:
            del self._ws_live[t.data_ptr()]
            return True
        return False

    def _release(self, t: torch.Tensor) -> None:
        """``t`` was read by a kernel that did not zero it: restore the zero invariant."""
        if self._ws_live.pop(t.data_ptr(), None) is not None:
            t.zero_()

    def silu_mul(self, gu, out_dtype=None):
        out_dtype = out_dtype or gu.dtype
        out = torch.empty(gu.shape[0], gu.shape[1] // 2, dtype=out_dtype, device=gu.device)
        zero = self._consumes(gu, out_dtype, gu.shape[1] % 8 == 0)
        self.ext.silu_mul(gu, out, zero)
        if not zero:
            self._release(gu)
        self.launches += 1
        return out

    # ------------------------------------------------------------------ matrix products
    def linear(self, a, w, bias=None, out_dtype=None, accumulate_into=None):
        """``a @ w.T (+ bias)``.

        out_dtype None asks for "an activation for the next kernel of this package": the compute
        dtype, or float32 sums where those come for free (the kernels that read activations take
        both; a float32 result may be an internal accumulation buffer that ``rope_kv_write`` or
        ``silu_mul`` clears as it reads it, so it must not be read again after that).
        With ``accumulate_into`` (a float32 tensor of the result's shape) the product may be
        added into that tensor instead; the return value is then None.
        """
        if a.dtype == torch.float32:
            if w.dtype != torch.float32:
                raise TypeError("float32 activations need float32 weights")
            out = torch.empty(a.shape[0], w.shape[0], dtype=torch.float32, device=a.device)
            self.ext.gemm_f32(a, w, bias, out)
            self.launches += 1
            return out if out_dtype in (None, torch.float32) else out.to(out_dtype)
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise TypeError(f"linear: unsupported dtypes {a.dtype} x {w.dtype}")
        T, K = a.shape
        N = w.shape[0]
        if self.use_skinny_gemm and T <= self.skinny_atomic_rows and K % 8 == 0:
            # few rows: the weights are streamed once through the tcgen05 kernel, work balanced
            # over all SMs, float32 sums added with atomics
            if out_dtype == torch.bfloat16:
                out = torch.empty(T, N, dtype=torch.bfloat16, device=a.device)
                self.ext.gemm_bf16_skinny(a, w, bias, out, False)
                self.launches += 1
                return out
            if accumulate_into is not None:
                self.ext.gemm_bf16_skinny(a, w, bias, accumulate_into, True)
                self.launches += 1
                return None
            out = (self._accumulator(T, N) if out_dtype is None
                   else torch.zeros(T, N, dtype=torch.float32, device=a.device))
            self.ext.gemm_bf16_skinny(a, w, bias, out, True)
            self.launches += 1
            return out
        if accumulate_into is not None and bias is None and self._addmm_in_place is not False:
            # many rows: the library adds the product into the residual stream (beta = 1)
            try:
                torch.addmm(accumulate_into, a, w.t(), out_dtype=torch.float32, out=accumulate_into)
                self._addmm_in_place = True
                return None
            except (RuntimeError, TypeError):
                if self._addmm_in_place:
                    raise
                self._addmm_in_place = False  # this build of the library cannot; use the plain form
        if out_dtype == torch.float32:
            out = torch.mm(a, w.t(), out_dtype=torch.float32)
            if bias is not None:
                out += bias.float()
            return out
        if bias is not None:
            return torch.addmm(bias, a, w.t())  # bias added before the one rounding to bfloat16
        return torch.mm(a, w.t())

    # ------------------------------------------------------------------ attention
    def rope_kv_write(self, qkv, *, num_heads, num_kv_heads, head_dim, positions, token_seq,
                      cos, sin, k_pages, v_pages, block_tables, page_tokens, out_dtype):
        """Rotate q and k, write k and v into their pages; returns the rotated queries."""
        zero = self._consumes(qkv, out_dtype, head_dim % 8 == 0)
        q = self.ext.rope_kv_write(qkv, num_heads, num_kv_heads, head_dim, positions, token_seq,
                                   cos, sin, k_pages, v_pages, block_tables, page_tokens,
                                   out_dtype == torch.bfloat16, zero)
        if not zero:
            self._release(qkv)
        self.launches += 1
        return q

    def attention_q_tile(self, dtype, head_dim):
        return int(self.ext.attention_q_tile(head_dim, dtype == torch.bfloat16,
                                             self.attention_kernel))

    def attention_plan(self, host_step, dtype, head_dim):
        """Work lists for this step: tiles of the portions, and the single-token sequences."""
        qt = self.attention_q_tile(dtype, head_dim)
        tiles, decode = [], []
        for s, n in enumerate(host_step.q_lens.tolist()):
            if n == 1:
                decode.append(s)
            else:
                tiles.extend((s, q0) for q0 in range(0, n, qt))
        # longest contexts first: their tiles run longest
        tiles.sort(key=lambda t: -(int(host_step.ctx_lens[t[0]]) - int(host_step.q_lens[t[0]]) + t[1]))
        return {
            "tiles": np.asarray(tiles, dtype=np.int32).reshape(-1, 2),
            "decode_seqs": np.asarray(decode, dtype=np.int32),
        }

    def decode_splits(self, num_decode, num_kv_heads, max_ctx):
        """Context partitions per (sequence, head): about six blocks per SM, 128 keys or more each
        (measured at one sequence of 2176 keys: 8 partitions 13.3 µs, 16 10.9, 28 11.9, 34 12.1)."""
        if num_decode == 0:
            return 1
        blocks = num_decode * num_kv_heads
        want = max(1, (6 * self.num_sms + blocks - 1) // blocks)
        return int(max(1, min(want, (max_ctx + 127) // 128, 64)))

    def paged_attention(self, q, *, num_heads, num_kv_heads, head_dim, scale, window, k_pages,
                        v_pages, block_tables, page_tokens, step, plan):
        out = torch.empty(q.shape[0], num_heads * head_dim, dtype=q.dtype, device=q.device)
        n_tiles = int(plan["tiles"].shape[0])
        n_dec = int(plan["decode_seqs"].shape[0])
        splits = step.decode_splits if step.decode_splits else self.decode_splits(
            n_dec, num_kv_heads, step.max_decode_ctx)
        scratch = None
        if n_dec and splits > 1:
            self.reserve_attention_scratch(head_dim, n_dec, num_heads, splits)
            scratch = self._scratch
        self.ext.paged_attention(
            q, out, k_pages, v_pages, num_heads, num_kv_heads, head_dim, float(scale),
            int(window), block_tables, step.ctx_lens, step.cu_q,
            plan["tiles"] if n_tiles else None, n_tiles,
            plan["decode_seqs"] if n_dec else None, n_dec, splits, scratch,
            self.attention_kernel,
        )
        self.launches += (1 if n_tiles else 0) + (1 if n_dec else 0)
        return out

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, top_k, top_p, min_p, seed, draw, kinds=3):
        """``kinds``: bit 0 = some row is greedy or cut by top-k / top-p / min-p, bit 1 = some row has
        a temperature and no cut; the kernel of a kind that is promised absent is not launched."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        rows = logits.shape[0]
        if self._sample_scratch is None or self._sample_rows < rows:
            if not torch.cuda.is_current_stream_capturing():
                # results of the blocks that share a row, and a counter per row (zero between launches)
                self._sample_rows = max(rows, 1024)
                self._sample_scratch = torch.zeros(int(self.ext.sample_scratch_ints(self._sample_rows)),
                                                   dtype=torch.int32, device=self.device)
        scratch = self._sample_scratch if self._sample_rows >= rows else None
        self.ext.sample(logits, temperature, top_k, top_p, min_p, seed, draw, out, scratch, kinds)
        self.launches += 1
        return out

    def logsumexp(self, logits):
        out = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
        self.ext.logsumexp(logits, out)
        self.launches += 1
        return out

    def apply_penalties(self, logits, row, token, count, presence, frequency, repetition):
        self.ext.apply_penalties(logits, row, token, count, presence, frequency, repetition)
        self.launches += 1

    def ban_tokens(self, logits, row, token):
        self.ext.ban_tokens(logits, row, token)
        self.launches += 1

    def token_state_add(self, state, slot, token, in_prompt):
        """Enter (slot, token) pairs into the penalties' token state ``[slots, vocab]`` (int32)."""
        self.ext.token_state_add(state, slot, token, in_prompt)
        self.launches += 1

    def apply_penalties_dense(self, logits, row, slot, presence, frequency, repetition, state):
        self.ext.apply_penalties_dense(logits, row, slot, presence, frequency, repetition, state)
        self.launches += 1


_instances: dict[str, CudaOps] = {}


def get_ops(device: torch.device | str = "cuda") -> CudaOps:
    key = str(torch.device(device))
    if key not in _instances:
        _instances[key] = CudaOps(device)
    return _instances[key]
