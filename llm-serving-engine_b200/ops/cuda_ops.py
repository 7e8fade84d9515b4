"""The kernel set of the product path: thin, checked calls into the sm_100a extension.

There is no other implementation behind these methods: if CUDA or the compiled extension is not
available, constructing :class:`CudaOps` raises.

Matrix products: float32 runs this package's own CUDA-core kernel (true 32-bit, no tensor-core
mode). bfloat16 products of up to 32 rows (decoding) run this package's tcgen05 kernel; with more
rows they go to cuBLAS through ``torch.mm`` with float32 accumulation, the same
library-for-linear-layers split as the reference (src/llmserve/models/layers.py:129-152).

The few-rows kernel shares a tile's K between blocks, which add their partial sums with integer
atomics into a buffer of 64-bit fixed-point numbers (value * 2^24). Such sums have the same bits
whatever the order of the additions was, so the bfloat16 path is reproducible from run to run.
The kernel that consumes the product (single-token attention, rotation and cache write, SiLU,
residual add and norm, or a plain conversion) reads the buffer, converts and leaves zeros behind. The buffers never leave
this class except as a :class:`PendingSums` that stands for "a product still to be added to the
residual stream".
"""

from __future__ import annotations

import numpy as np
import torch

from . import build

_DTYPES = (torch.float32, torch.bfloat16)


class PendingSums:
    """A product that is still to be added to the float32 tensor ``into`` (the residual stream).

    What a projection called with ``accumulate_into=x, may_defer=True`` may return instead of
    adding at once: the sums lie in a fixed-point buffer of the kernel set. Hand it, as the
    ``residual``, to the next ``add_rmsnorm`` on the same ``x`` (which adds it while it reads it
    anyway), or call :meth:`resolve` to have it added now. Exactly one of the two must happen
    before anything else reads ``x``.
    """

    __slots__ = ("ops", "sums", "into")

    def __init__(self, ops: "CudaOps", sums: torch.Tensor, into: torch.Tensor) -> None:
        self.ops, self.sums, self.into = ops, sums, into

    def resolve(self) -> None:
        """Add the sums to ``into`` now. Returns None: nothing is pending any more."""
        if self.sums is not None:
            self.ops.ext.fixed_to_float(self.sums, self.into, True)
            self.ops.launches += 1
            self.ops._sums_taken(self.sums)
            self.sums = None
        return None


# Cost of a block of the single-token attention kernel in units of one key: its start (tables,
# queries, first tile) and end (partial results, counter), and what each further partition adds
# to the merge. From timings at 2118 keys of head size 64: a wave of blocks takes about 39 ns per
# key and 5 us besides.
_BLOCK_START_KEYS = 130
_MERGE_KEYS_PER_SPLIT = 4


def choose_decode_splits(pairs: int, max_ctx: int, num_sms: int, blocks_per_sm: int) -> int:
    """Context partitions per (sequence, key/value head) for ``pairs`` such pairs.

    The kernel runs one block per (partition, pair); ``blocks_per_sm * num_sms`` of them run at a
    time, a *wave*. One tile of keys is in flight per warp, so a block's speed is set by latency,
    not by how many blocks share the SM, and a wave that is part empty takes as long as a full
    one: 12 sequences x 32 heads cut in 3 make 1152 blocks for 1036 places and took 49 us where
    24 sequences took 79. So the number of partitions is the one that minimises
    ``waves * (keys per block + a block's fixed cost)``, among partitions of 128 keys or more
    (measured at one sequence of 2176 keys: 8 partitions 13.3 us, 16 10.9, 28 11.9, 34 12.1).
    The context is rounded up to a power of two first, so that the choice (which captured graphs
    are keyed on) does not flicker from step to step. Without a known occupancy: about six blocks
    per SM.
    """
    if pairs <= 0:
        return 1
    most = int(max(1, min((max_ctx + 127) // 128, 64)))
    if blocks_per_sm <= 0:
        want = max(1, (6 * num_sms + pairs - 1) // pairs)
        return int(min(want, most))
    wave = blocks_per_sm * num_sms
    ctx = 1 << max(0, int(max_ctx) - 1).bit_length()

    def cost(s: int) -> int:
        waves = -(-pairs * s // wave)
        return waves * (-(-ctx // s) + _BLOCK_START_KEYS + _MERGE_KEYS_PER_SPLIT * s)

    return min(range(1, most + 1), key=lambda s: (cost(s), s))


class CudaOps:
    name = "cuda-sm100a"
    defers_adds = True  # linear(..., accumulate_into=x, may_defer=True) may return PendingSums

    def __init__(self, device: torch.device | str = "cuda") -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise RuntimeError(
                "llmserve_b200 runs on a CUDA device only (built for sm_100a); no CPU fallback exists"
            )
        self.ext = build.load_core()
        self._attn_loaded: set[int] = set()
        self._scratch: torch.Tensor | None = None
        self.decode_blocks_per_sm = 0  # of the single-token attention kernel; 0: not asked yet
        self.fuse_rotation_into_attention = True  # single tokens: attention makes q, k, v from the product's sums
        self._takes_sums_known: dict[tuple, bool] = {}
        self._sample_scratch: torch.Tensor | None = None
        self._sample_rows = 0
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        # 0: fastest available; 1: CUDA cores; 2: mma.sync fed by plain loads; 3: single tokens fed by TMA
        self.attention_kernel = 0  # (tests compare them)
        self.use_skinny_gemm = True
        # rows up to which the own tcgen05 product runs (measured: above it the library is faster)
        self.skinny_max_rows = int(self.ext.gemm_bf16_skinny_max_rows())
        # Fixed-point sum buffers of the few-rows product, by shape. A buffer is zero whenever it
        # is not in _sums_live (the kernel that takes a product's sums leaves zeros behind).
        self._sums: dict[tuple[int, int], torch.Tensor] = {}
        self._sums_live: set[int] = set()  # data_ptr of buffers whose sums have not been taken yet
        self._addmm_in_place: bool | None = None  # whether torch.addmm can add into a float32 tensor
        self.launches = 0  # kernels of this package enqueued (library matrix products not counted)

    # ------------------------------------------------------------------ capabilities
    def branch_dtype(self, dtype: torch.dtype) -> torch.dtype:
        """Dtype in which projections that feed the residual stream return their result."""
        return torch.float32

    def check_attention_shape(self, head_dim: int, dtype: torch.dtype, num_heads: int | None = None,
                              num_kv_heads: int | None = None) -> None:
        """Load the kernels of this head size. With the head counts given, also ask how many blocks
        of the single-token kernel an SM holds (the smallest answer over a model's layers is kept:
        :meth:`decode_splits` fills whole waves of that many blocks)."""
        if dtype not in _DTYPES:
            raise ValueError(f"attention kernels exist for float32 and bfloat16, not {dtype}")
        if head_dim not in self._attn_loaded:
            self.ext.load_attention_library(build.attention_library(head_dim), head_dim)
            self._attn_loaded.add(head_dim)
        if num_heads and num_kv_heads:
            n = int(self.ext.attention_decode_blocks_per_sm(head_dim, dtype == torch.bfloat16,
                                                            num_heads, num_kv_heads))
            if n > 0:
                self.decode_blocks_per_sm = min(self.decode_blocks_per_sm or n, n)

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
        """``residual`` may be a :class:`PendingSums` for ``x``: its sums are added as they are read."""
        sums = None
        if isinstance(residual, PendingSums):
            if residual.into is not x:
                raise ValueError("these pending sums belong to another tensor")
            if rows is None and out_dtype == torch.bfloat16 and x.shape[1] % 4 == 0 and residual.sums is not None:
                sums, residual.sums = residual.sums, None
                residual = sums
            else:  # only some rows are read here, so the whole product is added first
                residual = residual.resolve()
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device)
        self.ext.add_rmsnorm(x, residual, weight, float(eps), out, rows)
        self.launches += 1
        if sums is not None:
            self._sums_taken(sums)
        return out

    # ------------------------------------------------------------------ fixed-point sums
    def _product_sums(self, a, w, bias) -> torch.Tensor:
        """``a @ w.T (+ bias)`` as fixed-point sums in a buffer that the caller must have taken
        (by a kernel that clears it) before the buffer of this shape is used again."""
        T, N = a.shape[0], w.shape[0]
        buf = self._sums.get((T, N))
        if buf is None and not torch.cuda.is_current_stream_capturing():
            buf = self._sums[(T, N)] = torch.zeros(T, N, dtype=torch.int64, device=self.device)
        if buf is None or buf.data_ptr() in self._sums_live:
            buf = torch.zeros(T, N, dtype=torch.int64, device=self.device)  # rare: the shape's buffer is busy
        self._sums_live.add(buf.data_ptr())
        self.ext.gemm_bf16_skinny(a, w, bias, buf)
        self.launches += 1
        return buf

    def _sums_taken(self, buf: torch.Tensor) -> None:
        self._sums_live.discard(buf.data_ptr())

    def silu_mul(self, gu, out_dtype=None):
        out_dtype = out_dtype or gu.dtype
        out = torch.empty(gu.shape[0], gu.shape[1] // 2, dtype=out_dtype, device=gu.device)
        self.ext.silu_mul(gu, out)
        self.launches += 1
        return out

    # ------------------------------------------------------------------ matrix products
    def _few_rows(self, a, w) -> bool:
        """Does the own tcgen05 kernel serve this product?"""
        return (self.use_skinny_gemm and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and a.shape[0] <= self.skinny_max_rows and a.shape[1] % 8 == 0)

    def linear(self, a, w, bias=None, out_dtype=None, accumulate_into=None, may_defer=False):
        """``a @ w.T (+ bias)`` as a new tensor of ``out_dtype`` (None: the compute dtype).

        With ``accumulate_into`` (a float32 tensor of the result's shape) the product may be
        added into that tensor instead; the return value is then None. A caller that passes
        ``may_defer=True`` may get a :class:`PendingSums` instead, which it has to hand on to
        whoever reads ``accumulate_into`` next.
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
        T = a.shape[0]
        N = w.shape[0]
        if self._few_rows(a, w):
            # few rows: the weights are streamed once through the tcgen05 kernel, work balanced
            # over all SMs, partial sums added as fixed-point numbers
            sums = self._product_sums(a, w, bias)
            if accumulate_into is not None:
                pending = PendingSums(self, sums, accumulate_into)
                return pending if may_defer else pending.resolve()
            out = torch.empty(T, N, dtype=out_dtype or torch.bfloat16, device=a.device)
            self.ext.fixed_to_float(sums, out, False)
            self.launches += 1
            self._sums_taken(sums)
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

    def gated_silu(self, h, w, bias=None, out_dtype=None):
        """``silu(h @ gate.T) * (h @ up.T)`` for ``w = [gate rows; up rows]``. With few bfloat16
        rows the gate meets its activation as a float32 value (the activation kernel takes the
        product's fixed-point sums); otherwise as the product's rounded output."""
        out_dtype = out_dtype or h.dtype
        if self._few_rows(h, w) and out_dtype == torch.bfloat16 and w.shape[0] % 8 == 0:
            sums = self._product_sums(h, w, bias)
            out = self.silu_mul(sums, out_dtype=out_dtype)
            self._sums_taken(sums)
            return out
        return self.silu_mul(self.linear(h, w, bias), out_dtype=out_dtype)

    def project_rope_kv_write(self, h, w, bias, *, num_heads, num_kv_heads, head_dim, positions,
                              token_seq, cos, sin, k_pages, v_pages, block_tables, page_tokens,
                              out_dtype):
        """The fused q|k|v projection of ``h``, rotation of q and k, and the write of k and v into
        their pages; returns the rotated queries. With few bfloat16 rows q, k and v reach the
        rotation as float32 values (the rotation kernel takes the product's fixed-point sums)."""
        kw = dict(num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                  positions=positions, token_seq=token_seq, cos=cos, sin=sin, k_pages=k_pages,
                  v_pages=v_pages, block_tables=block_tables, page_tokens=page_tokens, out_dtype=out_dtype)
        if self._few_rows(h, w) and out_dtype == torch.bfloat16 and head_dim % 8 == 0:
            sums = self._product_sums(h, w, bias)
            q = self.rope_kv_write(sums, **kw)
            self._sums_taken(sums)
            return q
        return self.rope_kv_write(self.linear(h, w, bias), **kw)

    def project_attend(self, h, w, bias, *, num_heads, num_kv_heads, head_dim, scale, window, positions,
                       token_seq, cos, sin, k_pages, v_pages, writes, block_tables, page_tokens, step,
                       plan, out_dtype):
        """The fused q|k|v projection of ``h``, rotation, cache write (if ``writes``) and attention
        over the cache. For a step of few single tokens in bfloat16 this is two launches: the
        product leaves fixed-point sums, and the attention kernel makes its queries and this
        step's key and value from them (a single token's position is its context length - 1).
        Otherwise: projection, rotation + cache write, attention."""
        T = h.shape[0]
        n_dec = int(plan["decode_seqs"].shape[0])
        if (self.fuse_rotation_into_attention and writes and n_dec == T and int(plan["tiles"].shape[0]) == 0
                and self._few_rows(h, w) and out_dtype == torch.bfloat16 and self.attention_kernel in (0, 2)
                and self._takes_sums(head_dim, num_heads, num_kv_heads)):
            sums = self._product_sums(h, w, bias)
            out = torch.empty(T, num_heads * head_dim, dtype=out_dtype, device=h.device)
            splits = step.decode_splits if step.decode_splits else self.decode_splits(
                n_dec, num_kv_heads, step.max_decode_ctx)
            scratch = None
            if splits > 1:
                self.reserve_attention_scratch(head_dim, n_dec, num_heads, splits)
                scratch = self._scratch
            self.ext.paged_attention_from_sums(
                sums, out, k_pages, v_pages, num_heads, num_kv_heads, head_dim, float(scale), int(window),
                block_tables, step.ctx_lens, step.cu_q, plan["decode_seqs"], splits, scratch, cos, sin)
            self._sums_taken(sums)
            self.launches += 1
            return out
        q = self.project_rope_kv_write(
            h, w, bias, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
            positions=positions, token_seq=token_seq, cos=cos, sin=sin,
            k_pages=k_pages if writes else None, v_pages=v_pages if writes else None,
            block_tables=block_tables, page_tokens=page_tokens, out_dtype=out_dtype)
        return self.paged_attention(
            q, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale, window=window,
            k_pages=k_pages, v_pages=v_pages, block_tables=block_tables, page_tokens=page_tokens,
            step=step, plan=plan)

    def _takes_sums(self, head_dim, num_heads, num_kv_heads) -> bool:
        key = (head_dim, num_heads, num_kv_heads)
        if key not in self._takes_sums_known:
            self._takes_sums_known[key] = bool(self.ext.attention_takes_sums(head_dim, True, num_heads, num_kv_heads))
        return self._takes_sums_known[key]

    # ------------------------------------------------------------------ attention
    def rope_kv_write(self, qkv, *, num_heads, num_kv_heads, head_dim, positions, token_seq,
                      cos, sin, k_pages, v_pages, block_tables, page_tokens, out_dtype):
        """Rotate q and k, write k and v into their pages; returns the rotated queries."""
        q = self.ext.rope_kv_write(qkv, num_heads, num_kv_heads, head_dim, positions, token_seq,
                                   cos, sin, k_pages, v_pages, block_tables, page_tokens,
                                   out_dtype == torch.bfloat16)
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
        """Context partitions per (sequence, head) for a step of single tokens."""
        return choose_decode_splits(num_decode * num_kv_heads, max_ctx, self.num_sms, self.decode_blocks_per_sm)

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
