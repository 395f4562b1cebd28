"""The kernel set of the engine: thin bindings of the C entry points in ``csrc/``.

Every method takes torch tensors on the CUDA device, checks what the C side cannot
(dtypes, contiguity, shapes), and launches on torch's current stream.  There is no
fallback: if the device or the compiled library is missing, construction fails.

The kernel set's calling convention (also implemented by the plain PyTorch
statement in the tests):

pack_linear(w) -> w'                         a product's weight in the layout the kernels want
pack_gate_up(gate, up) -> w'                 the stacked gate/up weight
embed(table, token_ids, out)                 out[t] = float32(table[token_ids[t]])
rmsnorm(x, weight, eps, out, rows=None)      out[r] = norm(x[rows[r]] or x[r]), rounded to out.dtype
linear(a, w, out, accumulate=False)          out (+)= a @ w.T in float32
linear_xielu(h, w, ap, aq, out)              out = xielu(h @ w.T), one launch for few rows
glu_ffn(h, w_gate_up, w_down, residual, ...) residual += act(gate, up) @ w_down.T with a gated activation
gate_up_swiglu(h, w, out)                    out = silu(h @ gate.T) * (h @ up.T)
qk_norm_rope_store(qkv, ..., rotation, ...)  q/k head norm, rotation, k/v into pages, q out
qkv_rope_store(h, w, ..., rotation, ...)     the QKV product followed by qk_norm_rope_store, in one
                                             launch where the kernels can (step.scratch holds what
                                             they derive from the step, for one forward pass).
                                             ``rotation`` is what the position part answers
                                             (parts.rope.Rotation); kinds without a kernel are
                                             refused unless register_rotation gave a handler
step_lists(act_dtype)                        the host-built lists its kernels want of every step
paged_attention(...)                         causal attention over the pages of each token's request
                                             (single-token rows by flash-decoding, prompt portions by
                                             a prompt kernel, side by side where both are there)
qkv_attention(h, w, ..., out, ...)           qkv_rope_store followed by paged_attention, for a mixer
                                             that wants both at once
argmax(logits, out) / sample(...)            next token per row
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import load_library
from .mixer_ops import MixerOps
from .state_ops import StateOps

_CODE = {torch.float32: 0, torch.bfloat16: 1}
_vp = ctypes.c_void_p
_i = ctypes.c_int
_f = ctypes.c_float


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not float32 or bfloat16") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


MAX_KEY_RUNS = 8            # csrc/attn_prefill_tc.cu takes at most this many runs per tile


def choose_prompt_attention(n_tiles: int, num_heads: int, num_sms: int, *, reach: int = 1, window: int = 0,
                            two_heads_ok: bool = True, pairs_from: Optional[int] = 3, cut_keys: bool = True,
                            decode_blocks: Optional[int] = None, decode_blocks_per_sm: int = 4):
    """Which tcgen05 prompt-attention kernel takes a step's portions, and into how many runs the
    keys of every tile are cut: ``(two heads per block?, runs)``.  It depends on the step's shape
    alone (``reach``: ``StepBatch.portion_reach``), never on its data.

    * Many tiles per SM (``pairs_from`` (tile, head) pairs per SM or more): two heads of a kv
      group per block, uncut.
    * Portions that reach far back (``reach`` 2, no window): every block walks a long row of
      keys, where the two-heads kernel's shorter time per head and tile counts and its longer
      start does not (2,048 tokens at a context of 16,384: 350 -> 287 us; at 4,096 the two are
      equal, below it the one-head kernel wins); with fewer blocks than SMs it cuts the keys.
    * Fewer (tile, head) pairs than SMs and rows of more than a few key tiles (``reach`` 1):
      every tile's keys in as many runs as fill the SMs once, a block each, added by a second
      launch.  With two heads per block a run of a tile takes about 1.5 times as long and there
      may be twice as many runs; measured, that pays from four runs on (a 512-token portion at a
      context of 16,384: 101 -> 87 us), while two runs of two heads against the uncut one-head
      kernel lose at short contexts (1,024 tokens at 2,048: 28 -> 34 us).
    * ``decode_blocks`` (flash-decoding runs beside the prompt kernel): if all of its blocks
      find room on the SMs that the uncut one-head kernel leaves free, the keys stay uncut and
      that kernel's time hides behind them.
    """
    def runs_for(blocks: int) -> int:
        return max(1, min(MAX_KEY_RUNS, num_sms // max(1, blocks)))

    pairs = n_tiles * num_heads
    two = pairs_from is not None and two_heads_ok and pairs >= pairs_from * num_sms
    runs = 1
    if not two and two_heads_ok and reach == 2 and not window and pairs_from is not None:
        two = True
        if cut_keys:
            runs = runs_for(pairs // 2)
    elif not two and cut_keys and reach >= 1 and pairs < num_sms:
        runs = runs_for(pairs)
        runs2 = runs_for(pairs // 2) if two_heads_ok else 0
        if runs2 > 1.5 * runs and runs2 >= 4:
            two, runs = True, runs2
        if decode_blocks is not None and runs > 1 and decode_blocks <= (num_sms - pairs) * decode_blocks_per_sm:
            two, runs = False, 1
    return two, runs


class CudaOps(MixerOps, StateOps):
    name = "cuda"

    def __init__(self, device):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError(
                "the engine runs on a CUDA device only (there is no CPU path); "
                f"device {device!r} is not usable here")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(
                f"the kernels are built for sm_100a; device {device!r} is sm_{major}{minor}")
        self.core = load_library("core")
        self.core.ti_last_error.restype = ctypes.c_char_p
        self._declare()
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._bf16 = None
        self._gated = None
        self._rev4 = {}
        self.use_tc_biased_attention = True   # tensor-core kernels of the attention with a distance bias
        self.use_tcgen05_biased_attention = True   # ... its prompt portions on tcgen05 where the head size is 128
        self.grouped_experts_from = 128       # (token, slot) pairs from which the experts run as grouped products
        self.tcgen05_experts_from = 1024      # ... and from which those products run on tcgen05
        self.shared_rides_to = 1 << 17        # elements of a shared expert's matrix up to which it rides along
        self._counters = None
        self.use_tc_attention = True      # tcgen05 prompt attention where the shape allows
        self.use_2sm_gemm = True          # pairs of SMs for products with enough 256 x 256 tiles
        # (from about a third of the pairs busy on: a gate/up product of 512 rows, 48 pair tiles,
        # takes 10.5 against 12.6 us; at 32 pair tiles and fewer the one-SM kernel is ahead)
        self.pair_min_tiles = torch.cuda.get_device_properties(self.device).multi_processor_count * 3 // 10
        self.fuse_qkv_epilogue = True     # the prompt QKV product norms, rotates and stores its heads
        # steps of single tokens: flash-decoding norms, rotates and stores by itself, one launch less
        # per layer.  Off: measured equal to the separate kernels within 1 % at batch 8 and 4 %
        # slower at batch 1 (the work moves onto the attention kernel's own critical path)
        self.fuse_decode_rope = False
        # few-rows products on tcgen05 with K split over blocks: for weights of more than this many
        # bytes (None: never); up to it the direct-to-register kernel's shorter chain wins (measured:
        # a 4096 x 4096 weight takes 8.7 against 11.1 us at one row and 21 against 31 us at 64,
        # larger weights gain 15-50 % on tcgen05)
        self.few_tc_min_bytes = 1 << 25
        self._few_tickets = None
        # prompt attention with two heads per block (csrc/attn_prefill_tc2.cu) from this many
        # (head, tile) pairs per SM on (None: never)
        self.tc_attention_pairs_from = 3
        # a step's single-token rows and its prompt portions: flash-decoding beside the tcgen05
        # prompt kernel instead of behind it
        self.attention_side_by_side = True
        # a step with fewer (tile, head) pairs of prompt attention than SMs: the keys of every
        # tile cut into runs, one block each, added by a second launch
        self.split_prompt_keys = True
        # a product of many rows whose output has few tiles (a short prompt portion into a narrow
        # output): K cut into runs, added by a second launch
        self.split_k_portions = True
        # ... and when the norm of the output follows at once (``may_defer``), that norm adds the
        # runs as it reads its rows: one launch and one pass over the rows less
        self.norm_adds_runs = True
        self._pending_runs = None         # (scratch, runs, out, accumulate) of a product whose runs are not added yet
        # the feed-forward of a decode step of at most 16 rows as one launch, when a layer's
        # feed-forward weights fit into the GPU's shared memory (csrc/ffn_decode.cu); same bits as
        # the two products it replaces
        self.fuse_decode_ffn = True
        # ... and with the product in front of it that adds to the same residual (a mixer's output
        # projection, asked for with ``linear(..., may_defer=True)``) and the norm between them
        self.fuse_decode_tail = True
        self._ffn_counters = None
        self._pending = None              # a held-back ``out += a w^T`` (and the norm of ``out`` after it)
        self._retired = []                # outgrown counter buffers that captured graphs may still use
        # rotation kind -> handler(ops, qkv, q_weight, k_weight, eps, rotation, step, cache, q_out,
        # num_heads, num_kv_heads, head_dim) that norms, rotates and stores the heads of a float32
        # product; "neox" and "none" run on the kernels of csrc/, others are brought by parts
        self._rotations = CudaOps._ROTATIONS          # kinds are known to every kernel set
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # kernels launched so far: entry points called eagerly, plus, for every graph replay,
        # the entry points that were captured into that graph
        self.launches = 0

    # ---- plumbing ------------------------------------------------------------------------
    def _declare(self) -> None:
        c = self.core
        c.ti_embed.argtypes = [_vp, _i, _vp, _i, _i, _vp, _vp]
        c.ti_rmsnorm.argtypes = [_vp, _vp, _vp, _i, _i, _f, _vp, _i, _vp]
        c.ti_rmsnorm_merge.argtypes = [_vp, _vp, _i, _i, _vp, _i, _i, _f, _vp, _i, _vp]
        c.ti_swiglu.argtypes = [_vp, _i, _i, _i, _vp, _i, _vp]
        c.ti_argmax.argtypes = [_vp, _i, _i, _vp, _vp]
        c.ti_argmax_sliced.argtypes = [_vp, _i, _i, _vp, _vp, _vp, _vp]
        c.ti_gemm_simple.argtypes = [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]
        c.ti_qk_norm_rope_store.argtypes = [
            _vp, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i,
            _vp, _i, _vp, _vp]
        c.ti_paged_attention_simple.argtypes = [
            _vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp]
        c.ti_sample.argtypes = [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]
        c.ti_embed_sinusoid.argtypes = [_vp, _i, _vp, _vp, _vp, _f, _i, _i, _vp, _vp]
        c.ti_qkv_bias_norm_store.argtypes = [_vp, _i, _vp, _vp, _vp, _f, _vp, _vp, _vp, _i, _vp, _i, _i, _i,
                                             _i, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp]
        c.ti_attention_bias_simple.argtypes = [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i,
                                               _i, _i, _i, _i, _f, _vp, _i, _vp, _i, _vp, _vp, _vp]
        c.ti_router_topk.argtypes = [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp]
        c.ti_router_choose.argtypes = [_vp, _i, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp]
        c.ti_moe_gate_up_simple.argtypes = [_vp, _i, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _i, _i,
                                            _vp, _i, _f, _f, _i, _vp]
        c.ti_moe_down_simple.argtypes = [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp,
                                         _i, _vp, _vp]
        c.ti_scale_rows.argtypes = [_vp, _i, _i, _vp, _i, _i, _vp]

    @property
    def bf16(self):
        """The tensor-core kernels of the bfloat16 path, built and loaded when first needed."""
        if self._bf16 is None:
            b = load_library("bf16")
            b.ti_last_error.restype = ctypes.c_char_p
            b.ti_gemm_skinny.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp]
            b.ti_gemm_skinny_supported.argtypes = [_i, _i, _i, _i, _i]
            b.ti_gemm_skinny_xielu.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp]
            b.ti_ffn_decode_supported.argtypes = [_i] * 8
            b.ti_ffn_decode.argtypes = [_vp, _vp, _vp, _vp, _vp] + [_i] * 8 + [_vp, _vp, _vp]
            b.ti_attn_out_ffn_decode_supported.argtypes = [_i] * 10
            b.ti_attn_out_ffn_decode.argtypes = ([_vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp] + [_i] * 10
                                                 + [_vp, _vp, _vp])
            b.ti_gemm_tcgen05_few_supported.argtypes = [_i, _i, _i, _i, _i, _i]
            b.ti_gemm_tcgen05_few_scratch.argtypes = [_i, _i, _i, ctypes.POINTER(ctypes.c_longlong),
                                                      ctypes.POINTER(ctypes.c_int)]
            b.ti_gemm_tcgen05_few.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp,
                                              _vp, _vp]
            b.ti_attn_decode_supported.argtypes = [_i, _i, _i]
            b.ti_attn_decode_blocks_per_sm.argtypes = [_i]
            b.ti_attn_decode_fused.argtypes = [_vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i,
                                               _i, _i, _f, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp]
            b.ti_attn_decode_qkv_supported.argtypes = [_i, _i, _i]
            b.ti_attn_decode_qkv.argtypes = [_vp, _i, _vp, _vp, _f, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i,
                                             _i, _i, _i, _i, _i, _f, _i, _vp, _vp, _vp, _vp, _vp, _vp]
            b.ti_gemm_tcgen05.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp]
            b.ti_gemm_tcgen05_add_runs.argtypes = [_vp, _vp, _i, _i, _i, _i, _i, _vp]
            b.ti_gemm_tcgen05_splits.argtypes = [_i, _i, _i, _i]
            b.ti_gemm_tcgen05_supported.argtypes = [_i, _i, _i, _i, _i, _i, _i]
            b.ti_gemm_tcgen05_grouped.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp,
                                                  _vp, _vp]
            b.ti_gemm_tcgen05_grouped_glu.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _f,
                                                      _vp, _vp]
            b.ti_gemm_skinny_glu.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]
            b.ti_gemm_tcgen05_glu.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp]
            b.ti_gemm_tcgen05_2sm.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]
            qkv_args = [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i,
                        _i, _i, _vp, _vp, _vp]
            b.ti_gemm_tcgen05_qkv.argtypes = qkv_args
            b.ti_gemm_tcgen05_2sm_qkv.argtypes = qkv_args
            b.ti_rope_table.argtypes = [_vp, _vp, _i, _i, _vp, _vp]
            b.ti_attn_prefill_supported.argtypes = [_i, _i]
            b.ti_attn_prefill.argtypes = [_vp, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _f,
                                          _vp, _vp, _vp]
            b.ti_attn_prefill_tc_supported.argtypes = [_i, _i, _i, _i]
            b.ti_attn_prefill_tc.argtypes = [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i,
                                             _f, _vp, _i, _vp, _vp, _vp, _i, _vp]
            b.ti_attn_prefill_tc_splits.argtypes = [_i, _i]
            b.ti_attn_prefill_tc_merge.argtypes = [_vp, _i, _i, _i, _vp, _vp, _vp, _vp]
            b.ti_attn_prefill_tc2_supported.argtypes = [_i, _i, _i, _i]
            b.ti_attn_prefill_tc2.argtypes = b.ti_attn_prefill_tc.argtypes
            self._tile_rows = (int(b.ti_attn_prefill_tile_rows()), int(b.ti_attn_prefill_tc_tile_rows()))
            self._bf16 = b
        return self._bf16

    @property
    def gated(self):
        """The tensor-core kernels of the attention with a distance bias and of the routed
        feed-forward (bfloat16), built and loaded when first needed."""
        if self._gated is None:
            b = load_library("bf16_gated")
            b.ti_last_error.restype = ctypes.c_char_p
            b.ti_attn_bias_prefill_supported.argtypes = [_i, _i, _i]
            b.ti_attn_bias_prefill.argtypes = [_vp, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _f,
                                               _vp, _i, _vp, _i, _vp, _vp, _vp]
            b.ti_attn_bias_prefill_tc_supported.argtypes = [_i, _i, _i, _i, _i]
            b.ti_attn_bias_prefill_tc.argtypes = [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _f,
                                                  _vp, _i, _i, _vp, _i, _vp, _vp, _vp]
            b.ti_attn_bias_decode_supported.argtypes = [_i, _i, _i, _i]
            b.ti_attn_bias_decode.argtypes = [_vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _f,
                                              _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp]
            b.ti_moe_grouped_supported.argtypes = [_i, _i, _i]
            b.ti_moe_grouped.argtypes = [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp,
                                         _vp, _vp, _i, _i, _f, _f, _i, _vp]
            b.ti_moe_sort_padded.argtypes = [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]
            b.ti_moe_gather_scaled.argtypes = [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _vp]
            b.ti_moe_combine_rows.argtypes = [_vp, _vp, _i, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _vp]
            self._gated = b
        return self._gated

    def step_lists(self, act_dtype):
        """The host-built integer lists (``engine.batch.StepList``) that the attention kernels of
        this kernel set want in every step of an engine with activations of ``act_dtype``: the
        single-token rows, the rows of prompt portions, and the portions cut into tiles of each
        prompt-attention kernel's own height.  The 32-bit kernels need none."""
        if act_dtype != torch.bfloat16:
            return []
        from .step_lists import attention_lists, row_tile_lists
        self.bf16
        # ... and, where a mixer has announced attention with options, every entry cut into tiles
        # of as many tokens as that kernel's blocks take
        return attention_lists(self._tile_rows) + row_tile_lists(self._row_tile_tokens)

    def stream(self) -> int:
        """The CUDA stream (as an integer handle) on which the engine's kernels are launched; a
        part with kernels of its own launches on it too."""
        return self._stream()

    def launched(self, rc: int = 0, message: str = "") -> None:
        """Account for a launch made by a part's own library (and raise if it reports failure)."""
        self.launches += 1
        if rc != 0:
            raise KernelError(message or f"a part's kernel returned {rc}")

    def _stream(self) -> int:
        return torch._C._cuda_getCurrentRawStream(self._device_index)

    def _ok(self, rc: int, lib=None) -> None:
        self.launches += 1
        if rc != 0:
            raise KernelError((lib or self.core).ti_last_error().decode("utf-8", "replace"))

    def check_status(self) -> None:
        """Raise if a kernel has written the status word since the last check (a page id outside
        the pool, or a barrier wait that ran out)."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            if self._ffn_counters is not None:        # a wait that ran out leaves its round incomplete
                self._ffn_counters.zero_()
            meaning = {1: "a block-table entry named a page outside the pool",
                       2: "a bounded wait ran out (on a shared-memory barrier of a tensor-core kernel or "
                          "on the arrival counter of the fused feed-forward; the kernel gave up "
                          "instead of hanging; its output is not valid)"}.get(code, "unknown code")
            raise KernelError(f"a kernel reported device status {code}: {meaning}")

    def _grown(self, old, need: int, device):
        """A zeroed int32 buffer of at least ``need`` counters that replaces ``old``.  The old one
        stays alive: a captured graph still holds its address, and its launches still count in
        it and leave it at zero."""
        if old is not None:
            self._retired.append(old)
        return torch.zeros(max(4096, 2 * need), dtype=torch.int32, device=device)

    def _tc_gemm(self, m: int, n: int):
        """The tcgen05 product to use: on pairs of SMs when every pair gets a 256 x 256 tile."""
        tiles = -(-m // 256) * -(-n // 256)
        if self.use_2sm_gemm and tiles >= self.pair_min_tiles:
            return self.bf16.ti_gemm_tcgen05_2sm
        return self.bf16.ti_gemm_tcgen05

    def _run_tc_gemm(self, a, w, c, out_act, m, n, k, ldc, ld_act, mode, may_defer=False) -> None:
        """The tcgen05 product of many rows; an output of few tiles has its K cut into runs that a
        second launch adds (the one-SM kernel decides, this side brings the scratch)."""
        fn = self._tc_gemm(m, n)
        if fn is self.bf16.ti_gemm_tcgen05_2sm:
            self._ok(fn(a.data_ptr(), w.data_ptr(), _ptr(c), _ptr(out_act), m, n, k, a.stride(0), w.stride(0),
                        ldc, ld_act, mode, self.status.data_ptr(), self._stream()), self.bf16)
            return
        runs = int(self.bf16.ti_gemm_tcgen05_splits(m, n, k, mode)) if self.split_k_portions else 1
        ws = torch.empty(runs * m * n, dtype=torch.float32, device=a.device) if runs > 1 else None
        leave = bool(runs > 1 and may_defer and self.norm_adds_runs and c is not None and c.is_contiguous())
        self._ok(fn(a.data_ptr(), w.data_ptr(), _ptr(c), _ptr(out_act), m, n, k, a.stride(0), w.stride(0),
                    ldc, ld_act, mode, _ptr(ws), int(leave), self.status.data_ptr(), self._stream()), self.bf16)
        if leave:
            self._pending_runs = (ws, runs, c, mode == 1)
        elif runs > 1:
            self.launches += 1            # the launch that adds the runs

    def _few_tc(self, a, w, c, out_act, mode) -> bool:
        """Runs the split-K tcgen05 product for few rows if it applies to these operands."""
        m, k = a.shape
        n = w.shape[0]
        if (self.few_tc_min_bytes is None or m > 64 or n * k * 2 <= self.few_tc_min_bytes
                or a.data_ptr() % 16 or w.data_ptr() % 16
                or not self.bf16.ti_gemm_tcgen05_few_supported(m, n, k, a.stride(0), w.stride(0), mode)):
            return False
        ws_floats, tickets = ctypes.c_longlong(0), ctypes.c_int(0)
        self.bf16.ti_gemm_tcgen05_few_scratch(m, n, k, ctypes.byref(ws_floats), ctypes.byref(tickets))
        if self._few_tickets is None or self._few_tickets.numel() < tickets.value:
            self._few_tickets = self._grown(self._few_tickets, tickets.value, a.device)
        ws = torch.empty(ws_floats.value, dtype=torch.float32, device=a.device) if ws_floats.value else None
        self._ok(self.bf16.ti_gemm_tcgen05_few(
            a.data_ptr(), w.data_ptr(), _ptr(c), _ptr(out_act), m, n, k, a.stride(0), w.stride(0),
            c.stride(0) if c is not None else 0, out_act.stride(0) if out_act is not None else 0, mode,
            _ptr(ws), self._few_tickets.data_ptr(), self.status.data_ptr(), self._stream()), self.bf16)
        return True

    # ---- weights -------------------------------------------------------------------------
    def pack_linear(self, w: torch.Tensor) -> torch.Tensor:
        _code(w, "pack_linear")
        return w.contiguous()

    def pack_gate_up(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """Gate and up rows as one weight.  When the size allows, in strips of 16 rows: 8 gate
        rows followed by their 8 up rows, so that a product's epilogue holds both values of
        an output column and applies SwiGLU without a round trip through memory."""
        inter, k = gate.shape
        if gate.dtype == torch.bfloat16 and inter % 8 == 0:
            packed = torch.stack([gate.view(inter // 8, 8, k), up.view(inter // 8, 8, k)], dim=1)
            packed = packed.reshape(2 * inter, k).contiguous()
            packed._ti_interleaved = True
            return packed
        packed = torch.cat([gate, up], dim=0).contiguous()
        packed._ti_interleaved = False
        return packed

    # ---- rowwise -------------------------------------------------------------------------
    def embed(self, table, token_ids, out):
        _need(out.dtype == torch.float32 and out.is_contiguous(), "embed: out must be float32")
        _need(token_ids.dtype == torch.int32, "embed: token ids must be int32")
        self._ok(self.core.ti_embed(table.data_ptr(), _code(table, "embed"), token_ids.data_ptr(),
                                    token_ids.shape[0], table.shape[1], out.data_ptr(),
                                    self._stream()))

    def rmsnorm(self, x, weight, eps, out, rows=None):
        pr = self._pending_runs
        if pr is not None:
            self._pending_runs = None
            ws, runs, c, accumulate = pr
            rc = -1
            if (rows is None and x is c and out.dtype == torch.bfloat16 and out.is_contiguous()
                    and weight.dtype == torch.float32 and weight.shape[0] == x.shape[1] == out.shape[1]
                    and out.shape[0] == x.shape[0]):
                rc = self.core.ti_rmsnorm_merge(x.data_ptr(), ws.data_ptr(), runs, int(accumulate),
                                                weight.data_ptr(), x.shape[0], x.shape[1], float(eps),
                                                out.data_ptr(), _code(out, "rmsnorm"), self._stream())
            if rc == -1:                  # not a norm of that output, or sizes the fused form does not take
                self._add_runs(pr)
            else:
                self._ok(rc)
                return
        p = self._pending
        if p is not None:
            if (p.get("norm") is None and rows is None and x is p["out"] and out.dtype == torch.bfloat16
                    and weight.dtype == torch.float32 and weight.shape[0] == x.shape[1] == out.shape[1]
                    and x.is_contiguous() and out.is_contiguous() and out.shape[0] == x.shape[0]):
                p["norm"] = (weight, eps, out)
                return
            self.flush()
        _need(x.dtype == torch.float32 and x.is_contiguous(), "rmsnorm: x must be float32")
        _need(weight.dtype == torch.float32 and weight.shape[0] == x.shape[1],
              "rmsnorm: weight must be float32 of the row length")
        _need(out.is_contiguous() and out.shape[1] == x.shape[1], "rmsnorm: bad out")
        n_rows = x.shape[0] if rows is None else rows.shape[0]
        _need(out.shape[0] == n_rows, "rmsnorm: out has the wrong number of rows")
        if rows is not None:
            _need(rows.dtype == torch.int32, "rmsnorm: rows must be int32")
        self._ok(self.core.ti_rmsnorm(x.data_ptr(), weight.data_ptr(), _ptr(rows), n_rows,
                                      x.shape[1], float(eps), out.data_ptr(),
                                      _code(out, "rmsnorm"), self._stream()))

    def _add_runs(self, pr) -> None:
        ws, runs, c, accumulate = pr
        self._ok(self.bf16.ti_gemm_tcgen05_add_runs(ws.data_ptr(), c.data_ptr(), c.shape[0], c.shape[1],
                                                    c.stride(0), runs, int(accumulate), self._stream()), self.bf16)

    def flush(self) -> None:
        """Launch what ``linear(..., may_defer=True)`` and a norm after it have held back."""
        pr, self._pending_runs = self._pending_runs, None
        if pr is not None:
            self._add_runs(pr)
        p, self._pending = self._pending, None
        if p is None:
            return
        self.linear(p["a"], p["w"], p["out"], accumulate=True)
        if p.get("norm") is not None:
            weight, eps, normed = p["norm"]
            self.rmsnorm(p["out"], weight, eps, normed)

    def linear(self, a, w, out, accumulate=False, may_defer=False):
        """out (+)= a @ w.T.  With ``may_defer`` (and ``accumulate``) the kernel set may hold the
        product back and run it in one launch with a norm of ``out`` and a feed-forward into ``out``
        that follow immediately; any other operation of the kernel set, ``stream()`` and
        ``flush()`` launch it first.  The caller must not touch ``a`` or ``out`` by other means
        until then."""
        if self._pending is not None or self._pending_runs is not None:
            self.flush()
        m, k = a.shape
        n = w.shape[0]
        if (may_defer and accumulate and self.fuse_decode_tail and self.fuse_decode_ffn and m <= 16 and n <= 1024
                and a.dtype == w.dtype == torch.bfloat16 and out.dtype == torch.float32
                and w.shape[1] == k and tuple(out.shape) == (m, n)
                and a.stride(1) == w.stride(1) == out.stride(1) == 1):
            self._pending = {"a": a, "w": w, "out": out}
            return
        _need(w.shape[1] == k and tuple(out.shape) == (m, n), "linear: shapes do not agree")
        _need(out.dtype == torch.float32, "linear: out must be float32")
        _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1,
              "linear: rows must be contiguous")
        if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
            mode = 1 if accumulate else 0
            if self._few_tc(a, w, out, None, mode):
                return
            if self.bf16.ti_gemm_skinny_supported(m, n, k, a.stride(0), w.stride(0)):
                self._ok(self.bf16.ti_gemm_skinny(
                    a.data_ptr(), w.data_ptr(), out.data_ptr(), None, m, n, k, a.stride(0),
                    w.stride(0), out.stride(0), 0, mode, self._stream()), self.bf16)
                return
            if (m > 64 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and
                    out.data_ptr() % 16 == 0 and self.bf16.ti_gemm_tcgen05_supported(
                        m, n, k, a.stride(0), w.stride(0), out.stride(0), mode)):
                self._run_tc_gemm(a, w, out, None, m, n, k, out.stride(0), 0, mode, may_defer=may_defer)
                return
        self._ok(self.core.ti_gemm_simple(
            a.data_ptr(), _code(a, "linear"), w.data_ptr(), _code(w, "linear"), out.data_ptr(),
            m, n, k, a.stride(0), w.stride(0), out.stride(0), int(bool(accumulate)),
            self._stream()))

    def gate_up_swiglu(self, h, w_gate_up, out):
        inter = out.shape[1]
        _need(w_gate_up.shape[0] == 2 * inter, "gate_up_swiglu: weight must hold gate and up rows")
        interleaved = bool(getattr(w_gate_up, "_ti_interleaved", False))
        m, k = h.shape
        if (interleaved and h.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                and self._few_tc(h, w_gate_up, None, out, 2)):
            return
        if (interleaved and h.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                and self.bf16.ti_gemm_skinny_supported(m, 2 * inter, k, h.stride(0),
                                                       w_gate_up.stride(0))):
            self._ok(self.bf16.ti_gemm_skinny(
                h.data_ptr(), w_gate_up.data_ptr(), None, out.data_ptr(), m, 2 * inter, k,
                h.stride(0), w_gate_up.stride(0), 0, out.stride(0), 2, self._stream()), self.bf16)
            return
        if (interleaved and m > 64 and h.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                and inter % 8 == 0 and out.stride(0) % 8 == 0 and self.bf16.ti_gemm_tcgen05_supported(
                    m, 2 * inter, k, h.stride(0), w_gate_up.stride(0), 0, 2)):
            self._run_tc_gemm(h, w_gate_up, None, out, m, 2 * inter, k, 0, out.stride(0), 2)
            return
        gu = torch.empty((m, 2 * inter), dtype=torch.float32, device=h.device)
        self.linear(h, w_gate_up, gu)
        self._ok(self.core.ti_swiglu(gu.data_ptr(), m, inter, int(interleaved), out.data_ptr(),
                                     _code(out, "swiglu"), self._stream()))

    def linear_xielu(self, h, w, ap, aq, out):
        """out = xielu(h @ w.T) in the activation dtype: ``ap z^2 + z/2`` where ``z > 0``, ``aq (exp(z) -
        1 - z) + z/2`` elsewhere.  Few rows run as one launch (the product's epilogue applies the
        activation); otherwise the product is followed by ``xielu_rows``."""
        m, k = h.shape
        n = w.shape[0]
        _need(w.shape[1] == k and tuple(out.shape) == (m, n) and out.dtype == h.dtype
              and h.stride(1) == w.stride(1) == out.stride(1) == 1, "linear_xielu: shapes do not agree")
        if (h.dtype == w.dtype == torch.bfloat16 and h.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and (self.few_tc_min_bytes is None or n * k * 2 <= self.few_tc_min_bytes)
                and self.bf16.ti_gemm_skinny_supported(m, n, k, h.stride(0), w.stride(0))):
            self._ok(self.bf16.ti_gemm_skinny_xielu(h.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, h.stride(0),
                                                    w.stride(0), out.stride(0), float(ap), float(aq), self._stream()),
                     self.bf16)
            return
        z = torch.empty((m, n), dtype=torch.float32, device=h.device)
        self.linear(h, w, z)
        self.xielu_rows(z, ap, aq, out)

    def glu_ffn(self, h, w_gate_up, w_down, residual, kind, limit, alpha, row_scale=None):
        """residual += act(h Wgate^T, h Wup^T) Wdown^T with ``w_gate_up`` from pack_gate_up and the
        gated activation ``kind`` of ``glu_rows`` ("clamped": ``g = min(g, limit)``, ``u = clamp(u,
        -limit, limit)``, ``g sigmoid(alpha g) (u + 1)``); ``row_scale`` (float32, one per row)
        multiplies a row's activations."""
        from .state_ops import GLU_KINDS
        m, k = h.shape
        inter = w_down.shape[1]
        interleaved = bool(getattr(w_gate_up, "_ti_interleaved", False))
        y = torch.empty((m, inter), dtype=h.dtype, device=h.device)
        if (interleaved and h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and float(alpha) != 0.0
                and h.data_ptr() % 16 == 0
                and self.bf16.ti_gemm_skinny_supported(m, 2 * inter, k, h.stride(0), w_gate_up.stride(0))):
            # few rows: the activation in the epilogue of the product that streams the weights once
            self._ok(self.bf16.ti_gemm_skinny_glu(
                h.data_ptr(), w_gate_up.data_ptr(), y.data_ptr(), m, 2 * inter, k, h.stride(0), w_gate_up.stride(0),
                y.stride(0), GLU_KINDS[kind], float(limit), float(alpha), self._stream()), self.bf16)
        elif (interleaved and m > 64 and h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
                and inter % 8 == 0 and h.data_ptr() % 16 == 0 and self.bf16.ti_gemm_tcgen05_supported(
                    m, 2 * inter, k, h.stride(0), w_gate_up.stride(0), 0, 2)):
            # many rows: the activation in the epilogue of the tcgen05 product
            self._ok(self.bf16.ti_gemm_tcgen05_glu(
                h.data_ptr(), w_gate_up.data_ptr(), y.data_ptr(), m, 2 * inter, k, h.stride(0), w_gate_up.stride(0),
                y.stride(0), GLU_KINDS[kind], float(limit), float(alpha), self.status.data_ptr(), self._stream()),
                self.bf16)
        else:
            gu = torch.empty((m, 2 * inter), dtype=torch.float32, device=h.device)
            self.linear(h, w_gate_up, gu)
            self.glu_rows(gu, interleaved, kind, limit, alpha, y)
        if row_scale is not None:
            self.scale_rows(y, row_scale)
        self.linear(y, w_down, residual, accumulate=True)

    def swiglu_ffn(self, h, w_gate_up, w_down, residual, may_defer=False):
        """residual += (silu(h Wgate^T) * (h Wup^T)) Wdown^T, with ``w_gate_up`` from pack_gate_up.
        ``may_defer`` as for ``linear``: the last product may be held back (or its runs of K left
        unadded) for what follows, until the next operation or ``flush()``."""
        m, k = h.shape
        inter = w_down.shape[1]
        _need(w_gate_up.shape == (2 * inter, k) and w_down.shape[0] == residual.shape[1] == k
              and residual.shape[0] == m, "swiglu_ffn: shapes do not agree")
        y = torch.empty((m, inter), dtype=h.dtype, device=h.device)
        p = self._pending
        if p is not None:
            norm = p.get("norm")
            a, w_o = p["a"], p["w"]
            if (norm is not None and h is norm[2] and residual is p["out"]
                    and bool(getattr(w_gate_up, "_ti_interleaved", False))
                    and w_gate_up.dtype == w_down.dtype == torch.bfloat16
                    and w_gate_up.stride(1) == w_down.stride(1) == 1
                    and self.bf16.ti_attn_out_ffn_decode_supported(
                        m, k, inter, a.shape[1], a.stride(0), w_o.stride(0), w_gate_up.stride(0),
                        w_down.stride(0), y.stride(0), residual.stride(0))):
                self._pending = None
                if self._ffn_counters is None:
                    self._ffn_counters = self._grown(None, 4, h.device)
                self._ok(self.bf16.ti_attn_out_ffn_decode(
                    a.data_ptr(), w_o.data_ptr(), norm[0].data_ptr(), float(norm[1]), w_gate_up.data_ptr(),
                    w_down.data_ptr(), y.data_ptr(), residual.data_ptr(), m, k, inter, a.shape[1],
                    a.stride(0), w_o.stride(0), w_gate_up.stride(0), w_down.stride(0), y.stride(0),
                    residual.stride(0), self._ffn_counters.data_ptr(), self.status.data_ptr(),
                    self._stream()), self.bf16)
                return
            self.flush()
        if (self.fuse_decode_ffn and m <= 16 and bool(getattr(w_gate_up, "_ti_interleaved", False))
                and h.dtype == w_gate_up.dtype == w_down.dtype == torch.bfloat16
                and residual.dtype == torch.float32
                and h.stride(1) == w_gate_up.stride(1) == w_down.stride(1) == residual.stride(1) == 1
                and self.bf16.ti_ffn_decode_supported(m, k, inter, h.stride(0), w_gate_up.stride(0),
                                                      w_down.stride(0), y.stride(0), residual.stride(0))):
            if self._ffn_counters is None:
                self._ffn_counters = self._grown(None, 4, h.device)
            self._ok(self.bf16.ti_ffn_decode(
                h.data_ptr(), w_gate_up.data_ptr(), w_down.data_ptr(), y.data_ptr(), residual.data_ptr(),
                m, k, inter, h.stride(0), w_gate_up.stride(0), w_down.stride(0), y.stride(0),
                residual.stride(0), self._ffn_counters.data_ptr(), self.status.data_ptr(),
                self._stream()), self.bf16)
            return
        self.gate_up_swiglu(h, w_gate_up, y)
        self.linear(y, w_down, residual, accumulate=True, may_defer=may_defer)

    # ---- attention -----------------------------------------------------------------------
    def register_rotation(self, kind: str, handler) -> None:
        """Teach the kernel sets (all of them: the table belongs to the class) a rotation kind of a
        position part: ``handler(ops, qkv, q_weight,
        k_weight, eps, rotation, step, cache, q_out, num_heads, num_kv_heads, head_dim)`` gets the
        float32 QKV product and does what ``qk_norm_rope_store`` does for the built-in kinds."""
        self._rotations[kind] = handler

    def _rotation_handler(self, rotation):
        _need(getattr(rotation, "scale", 1.0) == 1.0,
              "these kernels turn heads without a factor on sine and cosine (rotation.scale must be 1)")
        try:
            return self._rotations[rotation.kind]
        except KeyError:
            raise KernelError(
                f"no kernel rotates heads the way {rotation.kind!r} asks; known kinds: "
                f"{', '.join(sorted(self._rotations))} (a part that brings its own registers a "
                f"handler with ops.register_rotation)") from None

    def qk_norm_rope_store(self, qkv, q_weight, k_weight, eps, rotation, step, cache, q_out,
                           num_heads, num_kv_heads, head_dim):
        self._rotation_handler(rotation)(self, qkv, q_weight, k_weight, eps, rotation, step, cache,
                                         q_out, num_heads, num_kv_heads, head_dim)

    def _rotate_builtin(self, qkv, q_weight, k_weight, eps, rotation, step, cache, q_out,
                        num_heads, num_kv_heads, head_dim):
        t = qkv.shape[0]
        _need(qkv.dtype == torch.float32 and qkv.stride(1) == 1, "qk_norm_rope_store: qkv float32")
        _need(qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim,
              "qk_norm_rope_store: qkv width does not match the head counts")
        rot, inv_freq = int(rotation.rotary_dim), rotation.inv_freq
        _need(0 <= rot <= head_dim and rot % 2 == 0,
              f"qk_norm_rope_store: rotated width {rot} must be even and at most head_dim {head_dim}")
        _need(rot == 0 or (inv_freq is not None and inv_freq.shape[0] == rot // 2
                           and inv_freq.dtype == torch.float32),
              "qk_norm_rope_store: the rotation table must hold rotary_dim/2 float32 values")
        pages, bt = cache.pages, cache.block_table
        _need(pages.is_contiguous() and tuple(pages.shape[1:]) ==
              (2, num_kv_heads, cache.page_size, head_dim), "qk_norm_rope_store: page layout")
        _need(bt.dtype == torch.int32 and bt.stride(1) == 1, "qk_norm_rope_store: block table int32")
        self._ok(self.core.ti_qk_norm_rope_store(
            qkv.data_ptr(), qkv.stride(0), q_weight.data_ptr(), k_weight.data_ptr(), float(eps),
            _ptr(inv_freq) if rot else None, step.positions.data_ptr(), step.req_of_tok.data_ptr(),
            bt.data_ptr(), bt.stride(0), pages.data_ptr(), _code(pages, "cache"), pages.shape[0],
            cache.page_size, int(bool(cache.writes)), t, num_heads, num_kv_heads, head_dim, rot,
            q_out.data_ptr(), _code(q_out, "q"), self.status.data_ptr(), self._stream()))

    def qkv_rope_store(self, h, w_qkv, q_weight, k_weight, eps, rotation, step, cache, q_out,
                       num_heads, num_kv_heads, head_dim):
        """``qk_norm_rope_store`` of ``h @ w_qkv.T``.  Prompt portions with head size 128 and a
        NeoX rotation over the whole head run as one tcgen05 product whose epilogue norms, rotates
        and stores each head, so the float32 product never reaches memory."""
        t = q_out.shape[0]
        pages, bt = cache.pages, cache.block_table
        self._rotation_handler(rotation)            # refuse an unknown kind before any launch
        inv_freq = rotation.inv_freq
        fused = (self.fuse_qkv_epilogue and t > 64 and head_dim == 128 and w_qkv.dtype == torch.bfloat16
                 and rotation.kind == "neox" and rotation.rotary_dim == head_dim
                 and self._rotations["neox"] is CudaOps._rotate_builtin
                 and q_out.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16
                 and h.dtype == torch.bfloat16
                 and w_qkv.stride(1) == 1 and w_qkv.stride(0) % 8 == 0 and w_qkv.shape[1] % 8 == 0
                 and w_qkv.data_ptr() % 16 == 0 and q_out.is_contiguous() and pages.is_contiguous()
                 and q_weight.data_ptr() % 16 == 0 and k_weight.data_ptr() % 16 == 0)
        if not fused:
            qkv = torch.empty((t, w_qkv.shape[0]), dtype=torch.float32, device=q_out.device)
            self.linear(h, w_qkv, qkv)
            self.qk_norm_rope_store(qkv, q_weight, k_weight, eps, rotation, step, cache, q_out,
                                    num_heads, num_kv_heads, head_dim)
            return
        n, k = w_qkv.shape
        _need(h.shape == (t, k) and h.stride(1) == 1 and n == (num_heads + 2 * num_kv_heads) * head_dim,
              "qkv_rope_store: shapes do not agree")
        _need(tuple(pages.shape[1:]) == (2, num_kv_heads, cache.page_size, head_dim),
              "qkv_rope_store: page layout")
        _need(bt.dtype == torch.int32 and bt.stride(1) == 1, "qkv_rope_store: block table int32")
        _need(inv_freq is not None and inv_freq.shape[0] == head_dim // 2 and inv_freq.dtype == torch.float32,
              "qkv_rope_store: the rotation table must hold head_dim/2 float32 values")
        key = ("rope_table", inv_freq.data_ptr())
        table = step.scratch.get(key)
        if table is None:                       # once per forward pass: the same for every layer
            table = torch.empty((t, 2, head_dim // 2), dtype=torch.float32, device=q_out.device)
            self._ok(self.bf16.ti_rope_table(step.positions.data_ptr(), inv_freq.data_ptr(), t,
                                             head_dim // 2, table.data_ptr(), self._stream()), self.bf16)
            step.scratch[key] = table
        fn = (self.bf16.ti_gemm_tcgen05_2sm_qkv if self._tc_gemm(t, n) is self.bf16.ti_gemm_tcgen05_2sm
              else self.bf16.ti_gemm_tcgen05_qkv)
        if h.data_ptr() % 16 or h.stride(0) % 8:
            h = h.contiguous()
        self._ok(fn(h.data_ptr(), w_qkv.data_ptr(), t, k, h.stride(0), w_qkv.stride(0),
                    q_weight.data_ptr(), k_weight.data_ptr(), float(eps), table.data_ptr(),
                    step.positions.data_ptr(), step.req_of_tok.data_ptr(), bt.data_ptr(), bt.stride(0),
                    pages.data_ptr(), pages.shape[0], cache.page_size, int(bool(cache.writes)),
                    num_heads, num_kv_heads, q_out.data_ptr(), self.status.data_ptr(), self._stream()),
                 self.bf16)

    def qkv_attention(self, h, w_qkv, q_weight, k_weight, eps, rotation, step, cache, out,
                      num_heads, num_kv_heads, head_dim, window, scale):
        """The whole front of an attention mixer: ``out = attention(rotate(norm(h @ w_qkv.T)))``
        with the new keys and values stored on the way (``qkv_rope_store`` followed by
        ``paged_attention``).  In a step of single-token rows the flash-decoding kernel takes the
        float32 product as it is and norms, rotates and stores by itself: one launch less."""
        t = h.shape[0]
        pages, bt = cache.pages, cache.block_table
        single = step.lists.get("single_rows")
        group = num_heads // num_kv_heads
        fused = (self.fuse_decode_rope and t > 0 and h.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                 and pages.dtype == torch.bfloat16 and single is not None and single.shape[0] == t
                 and rotation.kind == "neox" and rotation.rotary_dim == head_dim
                 and self._rotations["neox"] is CudaOps._rotate_builtin
                 and rotation.inv_freq is not None and rotation.inv_freq.dtype == torch.float32
                 and q_weight.dtype == torch.float32 and k_weight.dtype == torch.float32
                 and pages.is_contiguous() and out.is_contiguous()
                 and tuple(pages.shape[1:]) == (2, num_kv_heads, cache.page_size, head_dim)
                 and bt.dtype == torch.int32 and bt.stride(1) == 1
                 and self.bf16.ti_attn_decode_qkv_supported(head_dim, group, cache.page_size))
        if not fused:
            q = torch.empty((t, num_heads * head_dim), dtype=h.dtype, device=h.device)
            self.qkv_rope_store(h, w_qkv, q_weight, k_weight, eps, rotation, step, cache, q,
                                num_heads, num_kv_heads, head_dim)
            self.paged_attention(q, step, cache, out, num_heads, num_kv_heads, head_dim, window, scale)
            return
        width = w_qkv.shape[0]
        _need(width == (num_heads + 2 * num_kv_heads) * head_dim, "qkv_attention: weight rows")
        qkv = torch.empty((t, width), dtype=torch.float32, device=h.device)
        self.linear(h, w_qkv, qkv)
        splits = self.decode_splits(t, num_kv_heads, step.max_position or step.max_ctx_len, head_dim)
        part_o = torch.empty((t, num_heads, splits, head_dim), dtype=torch.float32, device=h.device)
        part_ml = torch.empty((t, num_heads, splits, 2), dtype=torch.float32, device=h.device)
        if self._counters is None or self._counters.numel() < t * num_kv_heads:
            self._counters = self._grown(self._counters, t * num_kv_heads, h.device)
        self._ok(self.bf16.ti_attn_decode_qkv(
            qkv.data_ptr(), width, q_weight.data_ptr(), k_weight.data_ptr(), float(eps),
            rotation.inv_freq.data_ptr(), single.data_ptr(), t, step.positions.data_ptr(),
            step.req_of_tok.data_ptr(), bt.data_ptr(), bt.stride(0), pages.data_ptr(), pages.shape[0],
            cache.page_size, int(bool(cache.writes)), num_heads, num_kv_heads, head_dim, int(window or 0),
            float(scale), splits, part_o.data_ptr(), part_ml.data_ptr(), self._counters.data_ptr(),
            out.data_ptr(), self.status.data_ptr(), self._stream()), self.bf16)

    def decode_splits(self, rows: int, num_kv_heads: int, max_position: int, head_dim: int = 128) -> int:
        """In how many blocks the keys of a decoding row are cut, per kv head.  It depends on
        the padded batch size and on the model's longest context only, so that a step cuts
        the same way whether it runs eagerly or from a graph."""
        bucket = 1
        while bucket < rows:
            bucket *= 2
        # one-warp blocks, as many per SM as shared memory allows: fill the GPU once, never more
        want = (self.bf16.ti_attn_decode_blocks_per_sm(head_dim) * self.num_sms) // (bucket * num_kv_heads)
        return max(1, min(want, -(-max_position // 64), 256))

    def paged_attention(self, q, step, cache, out, num_heads, num_kv_heads, head_dim, window,
                        scale):
        pages, bt = cache.pages, cache.block_table
        _need(q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype,
              "paged_attention: q and out must be contiguous and of one dtype")
        _need(pages.is_contiguous() and tuple(pages.shape[1:]) ==
              (2, num_kv_heads, cache.page_size, head_dim), "paged_attention: page layout")
        win = int(window or 0)
        rows, n_rows = None, q.shape[0]
        lists = step.lists
        tensor_cores = q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16
        if tensor_cores and "single_rows" not in lists:
            raise KernelError("paged_attention: the step was built without this kernel set's lists "
                              "(pass lists=ops.step_lists(dtype) to build_step_batch)")
        single = lists["single_rows"] if tensor_cores else None
        n_dec = single.shape[0] if tensor_cores else 0
        decode = bool(n_dec) and bool(self.bf16.ti_attn_decode_supported(
            head_dim, num_heads // num_kv_heads, cache.page_size))
        small, big = self._tile_rows if tensor_cores else (0, 0)
        tiles = lists[f"portion_tiles_{small}"] if tensor_cores else None
        prompt = (tensor_cores and tiles.shape[0] > 0
                  and bool(self.bf16.ti_attn_prefill_supported(head_dim, cache.page_size)))
        prompt_tc = prompt and self.use_tc_attention and bool(self.bf16.ti_attn_prefill_tc_supported(
            head_dim, cache.page_size, num_heads, num_kv_heads))
        # Single-token rows beside prompt portions: the two kernels need nothing of one another.
        # The prompt kernel (tensor-bound, on a part of the SMs) goes first and releases its
        # dependents only when its own wait has returned; flash-decoding (bound by HBM) then runs
        # beside it on what that wait covered and waits for the prompt kernel at its end.
        beside = decode and prompt_tc and self.attention_side_by_side

        def run_decode():
            splits = self.decode_splits(n_dec, num_kv_heads, step.max_position or step.max_ctx_len, head_dim)
            part_o = torch.empty((n_dec, num_heads, splits, head_dim), dtype=torch.float32,
                                 device=q.device)
            part_ml = torch.empty((n_dec, num_heads, splits, 2), dtype=torch.float32,
                                  device=q.device)
            if self._counters is None or self._counters.numel() < n_dec * num_kv_heads:
                # zero once; every launch leaves its counters at zero again
                self._counters = self._grown(self._counters, n_dec * num_kv_heads, q.device)
            self._ok(self.bf16.ti_attn_decode_fused(
                q.data_ptr(), single.data_ptr(), n_dec, step.positions.data_ptr(),
                step.req_of_tok.data_ptr(), bt.data_ptr(), bt.stride(0), pages.data_ptr(),
                pages.shape[0], cache.page_size, num_heads, num_kv_heads, head_dim, win,
                float(scale), splits, part_o.data_ptr(), part_ml.data_ptr(),
                self._counters.data_ptr(), out.data_ptr(), self.status.data_ptr(), int(beside),
                self._stream()), self.bf16)

        if decode and not beside:
            run_decode()
        if decode:
            rows, n_rows = lists["portion_rows"], lists["portion_rows"].shape[0]
            if n_rows == 0:
                return
        if prompt:
            if prompt_tc:
                tiles = lists[f"portion_tiles_{big}"]
                n_tiles = tiles.shape[0]
                pairs_ok = bool(self.bf16.ti_attn_prefill_tc2_supported(head_dim, cache.page_size, num_heads,
                                                                        num_kv_heads))
                decode_blocks = 0
                if beside:
                    decode_blocks = n_dec * num_kv_heads * self.decode_splits(
                        n_dec, num_kv_heads, step.max_position or step.max_ctx_len, head_dim)
                two, runs = choose_prompt_attention(
                    n_tiles, num_heads, self.num_sms, reach=getattr(step, "portion_reach", 1), window=win,
                    two_heads_ok=pairs_ok, pairs_from=self.tc_attention_pairs_from,
                    cut_keys=self.split_prompt_keys, decode_blocks=decode_blocks if beside else None,
                    decode_blocks_per_sm=int(self.bf16.ti_attn_decode_blocks_per_sm(head_dim)))
                part_o = part_ml = None
                if runs > 1:
                    part_o = torch.empty((n_tiles, num_heads, runs, big, head_dim), dtype=torch.float32,
                                         device=q.device)
                    part_ml = torch.empty((n_tiles, num_heads, runs, big, 2), dtype=torch.float32,
                                          device=q.device)
                kernel = self.bf16.ti_attn_prefill_tc2 if two else self.bf16.ti_attn_prefill_tc
                self._ok(kernel(
                    q.data_ptr(), q.shape[0], tiles.data_ptr(), n_tiles,
                    step.positions.data_ptr(), bt.data_ptr(), bt.stride(0), pages.data_ptr(),
                    pages.shape[0], cache.page_size, num_heads, num_kv_heads, head_dim, win,
                    float(scale), out.data_ptr(), runs, _ptr(part_o), _ptr(part_ml),
                    self.status.data_ptr(), int(beside), self._stream()), self.bf16)
                if beside:
                    run_decode()                   # (its last block waits for the prompt kernel)
                if runs > 1:
                    self._ok(self.bf16.ti_attn_prefill_tc_merge(
                        tiles.data_ptr(), n_tiles, num_heads, runs, part_o.data_ptr(), part_ml.data_ptr(),
                        out.data_ptr(), self._stream()), self.bf16)
            else:
                self._ok(self.bf16.ti_attn_prefill(
                    q.data_ptr(), tiles.data_ptr(), tiles.shape[0], step.positions.data_ptr(),
                    bt.data_ptr(), bt.stride(0), pages.data_ptr(), pages.shape[0], cache.page_size,
                    num_heads, num_kv_heads, head_dim, win, float(scale), out.data_ptr(),
                    self.status.data_ptr(), self._stream()), self.bf16)
            if rows is not None:          # the single-token rows went through the decode kernel
                return
            rows, n_rows = single, n_dec
            if n_rows == 0:
                return
        self._ok(self.core.ti_paged_attention_simple(
            q.data_ptr(), _code(q, "q"), _ptr(rows), step.positions.data_ptr(),
            step.req_of_tok.data_ptr(), bt.data_ptr(), bt.stride(0), pages.data_ptr(),
            _code(pages, "cache"), pages.shape[0], cache.page_size, n_rows, num_heads,
            num_kv_heads, head_dim, win, float(scale), out.data_ptr(), self.status.data_ptr(),
            self._stream()))

    # ---- attention with a distance bias, kept first tokens and an output gate ---------------
    def embed_sinusoid(self, table, token_ids, positions, freq, scale, out):
        """out[t] = float32(table[token_ids[t]]) * scale + wave(positions[t]); wave(p)[2i] =
        sin(p freq[i]), wave(p)[2i + 1] = cos(p freq[i]); ``freq`` None: no wave."""
        _need(out.dtype == torch.float32 and out.is_contiguous(), "embed_sinusoid: out must be float32")
        _need(token_ids.dtype == torch.int32 and positions.dtype == torch.int32,
              "embed_sinusoid: token ids and positions must be int32")
        _need(freq is None or (freq.dtype == torch.float32 and freq.shape[0] >= (table.shape[1] + 1) // 2),
              "embed_sinusoid: one float32 frequency per pair of columns")
        self._ok(self.core.ti_embed_sinusoid(table.data_ptr(), _code(table, "embed_sinusoid"),
                                             token_ids.data_ptr(), positions.data_ptr(), _ptr(freq),
                                             float(scale), token_ids.shape[0], table.shape[1],
                                             out.data_ptr(), self._stream()))

    def _reversed_bias(self, dist_bias):
        """The distance table as the tcgen05 prompt kernel reads it, made once per table:
        ``[heads, 4, pitch]`` float32, copy c of a head holding ``R[j + c]`` at ``j``, where
        ``R[k] = bias[clamp(n + 127 - k, 0, n - 1)]`` for ``k < n + 256`` (the table reversed, with 128
        entries of padding at both ends), so that a row's 128 entries of a key tile are one aligned,
        ascending run in one of the copies."""
        key = (dist_bias.data_ptr(), tuple(dist_bias.shape))
        found = self._rev4.get(key)
        if found is None:
            heads, n = dist_bias.shape
            pitch = (n + 256 + 4 + 3) // 4 * 4
            k = torch.arange(pitch + 3, device=dist_bias.device)
            r = dist_bias[:, (n + 127 - k).clamp(0, n - 1)]                      # [heads, pitch + 3]
            found = torch.stack([r[:, c:c + pitch] for c in range(4)], dim=1).contiguous()
            self._rev4[key] = (found, dist_bias)             # the table stays alive with its copy
            return found
        return found[0]

    @staticmethod
    def _page_elems(cache, num_kv_heads, dk, dv) -> int:
        return num_kv_heads * cache.page_size * (dk + dv)

    def qkv_bias_norm_store(self, proj, bias, q_weight, k_weight, eps, step, cache, q_out,
                            num_heads, num_kv_heads, dk, dv):
        """From the float32 product ``proj`` (columns: query heads, then, if the cache slot is
        written, key heads and value heads; anything behind them is left alone): add ``bias``,
        bring query and key heads to unit root mean square (times ``q_weight`` / ``k_weight`` if
        given), store keys and values in the token's page and the queries in ``q_out``."""
        t = proj.shape[0]
        pages, bt = cache.pages, cache.block_table
        writes = bool(cache.writes)
        need = num_heads * dk + (num_kv_heads * (dk + dv) if writes else 0)
        _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= need,
              "qkv_bias_norm_store: the product must be float32 and hold all heads")
        _need(bias is None or (bias.dtype == torch.float32 and bias.shape[0] >= need and bias.is_contiguous()),
              "qkv_bias_norm_store: bias must be float32, one value per column")
        _need(pages.is_contiguous() and pages[0].numel() == self._page_elems(cache, num_kv_heads, dk, dv),
              "qkv_bias_norm_store: page layout")
        _need(bt.dtype == torch.int32 and bt.stride(1) == 1, "qkv_bias_norm_store: block table int32")
        _need(q_out.is_contiguous() and tuple(q_out.shape) == (t, num_heads * dk), "qkv_bias_norm_store: q_out")
        self._ok(self.core.ti_qkv_bias_norm_store(
            proj.data_ptr(), proj.stride(0), _ptr(bias), _ptr(q_weight), _ptr(k_weight), float(eps),
            step.positions.data_ptr(), step.req_of_tok.data_ptr(), bt.data_ptr(), bt.stride(0),
            pages.data_ptr(), _code(pages, "cache"), pages.shape[0], cache.page_size, int(writes), t,
            num_heads, num_kv_heads, dk, dv, q_out.data_ptr(), _code(q_out, "q"),
            self.status.data_ptr(), self._stream()))

    def biased_attention(self, q, step, cache, out, num_heads, num_kv_heads, dk, dv, window, keep_first,
                         scale, dist_bias, gate):
        """Causal attention over the pages of each token's request: key ``j`` is visible to token
        ``i`` when ``i - j < window`` (no window: always) or ``j < keep_first``; the score is
        ``(q . k) * scale + dist_bias[head][min(i - j, last)]``; the normalised output is
        multiplied by ``sigmoid(gate)`` (``gate``: float32 ``[T, heads * dv]``, rows may be strided)."""
        pages, bt = cache.pages, cache.block_table
        t = q.shape[0]
        _need(q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype,
              "biased_attention: q and out must be contiguous and of one dtype")
        _need(tuple(q.shape) == (t, num_heads * dk) and tuple(out.shape) == (t, num_heads * dv),
              "biased_attention: shapes of q and out")
        _need(pages.is_contiguous() and pages[0].numel() == self._page_elems(cache, num_kv_heads, dk, dv),
              "biased_attention: page layout")
        _need(dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.is_contiguous()
                                    and dist_bias.shape[0] == num_heads),
              "biased_attention: the bias table must be float32 [heads, distances]")
        _need(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1
                               and tuple(gate.shape) == (t, num_heads * dv)),
              "biased_attention: the gate must be float32 [tokens, heads * dv]")
        rows, n_rows = None, t
        lists = step.lists
        if (self.use_tc_biased_attention and q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16
                and dist_bias is not None and "single_rows" in lists
                and (gate is None or (gate.stride(0) % 2 == 0 and gate.data_ptr() % 8 == 0))
                and self.gated.ti_attn_bias_prefill_supported(dk, dv, cache.page_size)):
            self.bf16
            tiles = lists[f"portion_tiles_{self._tile_rows[0]}"]
            big = lists.get(f"portion_tiles_{self._tile_rows[1]}")
            if (tiles.shape[0] and self.use_tcgen05_biased_attention and big is not None
                    and q.data_ptr() % 16 == 0 and out.data_ptr() % 32 == 0
                    and (gate is None or (gate.stride(0) % 4 == 0 and gate.data_ptr() % 16 == 0))
                    and tuple(pages.shape[1:]) == (2, num_kv_heads, cache.page_size, dk)
                    and self.gated.ti_attn_bias_prefill_tc_supported(dk, dv, cache.page_size, num_heads, num_kv_heads)):
                # head size 128: the tcgen05 kernel, on tiles of its own height
                rev4 = self._reversed_bias(dist_bias)
                self._ok(self.gated.ti_attn_bias_prefill_tc(
                    q.data_ptr(), q.shape[0], big.data_ptr(), big.shape[0], step.positions.data_ptr(), bt.data_ptr(),
                    bt.stride(0), pages.data_ptr(), pages.shape[0], cache.page_size, num_heads, num_kv_heads, dk,
                    int(window or 0), int(keep_first), float(scale), rev4.data_ptr(), dist_bias.shape[1],
                    rev4.shape[2], _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(),
                    self.status.data_ptr(), self._stream()), self.gated)
                rows = lists["single_rows"]
                n_rows = rows.shape[0]
                if n_rows == 0:
                    return
            elif tiles.shape[0]:
                self._ok(self.gated.ti_attn_bias_prefill(
                    q.data_ptr(), tiles.data_ptr(), tiles.shape[0], step.positions.data_ptr(), bt.data_ptr(),
                    bt.stride(0), pages.data_ptr(), pages.shape[0], cache.page_size, num_heads, num_kv_heads, dk,
                    int(window or 0), int(keep_first), float(scale), dist_bias.data_ptr(), dist_bias.shape[1],
                    _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(),
                    self.status.data_ptr(), self._stream()), self.gated)
                rows = lists["single_rows"]
                n_rows = rows.shape[0]
                if n_rows == 0:
                    return
            single = lists["single_rows"]
            if single.shape[0] and self.gated.ti_attn_bias_decode_supported(
                    dk, dv, num_heads // num_kv_heads, cache.page_size):
                # few rows: the keys of a row in several runs, a block each, so that the SMs are busy.
                # The count depends on the step's shape alone (padded rows, the model's bounds).
                n_single = single.shape[0]
                most_keys = step.max_position or step.max_ctx_len
                if window:
                    most_keys = min(most_keys, int(window) + int(keep_first))
                nsplit = max(1, min(2 * self.num_sms // max(1, n_single * num_kv_heads), -(-most_keys // 32) // 8, 64))
                part_o = part_ml = None
                if nsplit > 1:
                    part_o = torch.empty((n_single, num_heads, nsplit, dk), dtype=torch.float32, device=q.device)
                    part_ml = torch.empty((n_single, num_heads, nsplit, 2), dtype=torch.float32, device=q.device)
                    self.launches += 1
                self._ok(self.gated.ti_attn_bias_decode(
                    q.data_ptr(), single.data_ptr(), single.shape[0], step.positions.data_ptr(),
                    step.req_of_tok.data_ptr(), bt.data_ptr(), bt.stride(0), pages.data_ptr(), pages.shape[0],
                    cache.page_size, num_heads, num_kv_heads, dk, int(window or 0), int(keep_first),
                    float(scale), dist_bias.data_ptr(), dist_bias.shape[1], _ptr(gate),
                    gate.stride(0) if gate is not None else 0, out.data_ptr(), nsplit, _ptr(part_o),
                    _ptr(part_ml), self.status.data_ptr(), self._stream()), self.gated)
                return
        self._ok(self.core.ti_attention_bias_simple(
            q.data_ptr(), _code(q, "q"), _ptr(rows), step.positions.data_ptr(), step.req_of_tok.data_ptr(),
            bt.data_ptr(), bt.stride(0), pages.data_ptr(), _code(pages, "cache"), pages.shape[0],
            cache.page_size, n_rows, num_heads, num_kv_heads, dk, dv, int(window or 0), int(keep_first),
            float(scale), _ptr(dist_bias), dist_bias.shape[1] if dist_bias is not None else 0,
            _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(),
            self.status.data_ptr(), self._stream()))

    # ---- routed feed-forward ---------------------------------------------------------------
    def pack_experts(self, gate, up, down):
        """The stacked weights of a routed feed-forward (``[experts, ff, width]`` twice and
        ``[experts, width, ff]``) in the layout the kernels want: an expert's gate and up rows as
        one matrix (strips of 8 and 8 where the sizes allow, for the SwiGLU epilogues)."""
        _need(gate.dtype == up.dtype == down.dtype, "pack_experts: one dtype for all experts")
        _code(gate, "pack_experts")
        experts, ff, width = gate.shape
        interleaved = gate.dtype == torch.bfloat16 and ff % 8 == 0
        if interleaved:          # strips of 8 gate rows and their 8 up rows, as pack_gate_up lays them out
            gate_up = torch.stack([gate.view(experts, ff // 8, 8, width), up.view(experts, ff // 8, 8, width)], dim=2)
            gate_up = gate_up.reshape(experts, 2 * ff, width).contiguous()
        else:
            gate_up = torch.cat([gate, up], dim=1).contiguous()
        return {"gate_up": gate_up, "down": down.contiguous(), "interleaved": interleaved}

    def router_topk(self, logits, experts, top, ids, weights, shared_gate=None, softmax=False):
        """Per row the ``top`` largest of the first ``experts`` logits (ties: the lower index):
        ``ids`` int32 and ``weights = sigmoid(logit)`` float32, both ``[rows, top]``; with
        ``shared_gate`` also ``sigmoid(logits[:, experts])`` per row.  ``softmax``: the weights are
        the chosen experts' shares of the softmax over all ``experts`` logits, not renormalised."""
        t = logits.shape[0]
        _need(logits.dtype == torch.float32 and logits.stride(1) == 1
              and logits.shape[1] >= experts + (shared_gate is not None), "router_topk: float32 logits")
        _need(ids.dtype == torch.int32 and weights.dtype == torch.float32 and ids.is_contiguous()
              and weights.is_contiguous() and tuple(ids.shape) == tuple(weights.shape) == (t, top),
              "router_topk: ids int32 and weights float32, [rows, top]")
        self._ok(self.core.ti_router_topk(logits.data_ptr(), logits.stride(0), t, experts, top,
                                          experts if shared_gate is not None else -1, ids.data_ptr(),
                                          weights.data_ptr(), _ptr(shared_gate), int(bool(softmax)),
                                          self._stream()))

    def router_choose(self, logits, total, top, ids, weights, correction=None, groups=1, keep=1):
        """Per row, from the first ``total`` float32 logits: scores ``s = softmax(logits)``; the
        choice looks at ``s + correction`` (float32 ``[total]`` or None), only inside the ``keep`` of
        ``groups`` equal groups of neighbouring outputs whose largest such value is largest, and
        takes the ``top`` largest there (ties: the lower index).  ``ids`` int32 and ``weights``
        float32 ``[rows, top]``: the chosen outputs and their ``s``, not renormalised."""
        t = logits.shape[0]
        _need(logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= total,
              "router_choose: float32 logits")
        _need(correction is None or (correction.dtype == torch.float32 and correction.is_contiguous()
                                     and correction.shape[0] == total), "router_choose: one float32 correction per output")
        _need(ids.dtype == torch.int32 and weights.dtype == torch.float32 and ids.is_contiguous()
              and weights.is_contiguous() and tuple(ids.shape) == tuple(weights.shape) == (t, top),
              "router_choose: ids int32 and weights float32, [rows, top]")
        self._ok(self.core.ti_router_choose(logits.data_ptr(), logits.stride(0), t, int(total), int(top),
                                            _ptr(correction), int(groups), int(keep), ids.data_ptr(),
                                            weights.data_ptr(), self._stream()))

    def routed_experts(self, h, w, ids, weights, residual, shared=None, act=None, identity=False):
        """residual[t] += sum over slots s of Wdown_e (silu(w g) * (w u)), g = Wgate_e h[t],
        u = Wup_e h[t], e = ids[t, s], w = weights[t, s].  ``shared`` (may be None):
        ``(w_gate_up from pack_gate_up, w_down, gate)`` of an expert that every token uses, its
        output times ``gate[t]``: residual[t] += gate[t] * Wdown (silu(g) * u).  Few tokens run
        it inside the experts' two launches.  ``act`` (may be None: silu) names another gated
        activation, ``(kind, limit, alpha)`` as ``glu_rows`` takes them; the pair's weight then
        scales the expert's output, residual[t] += w Wdown_e act(g, u), and there is no ``shared``.
        ``identity``: an index at or behind the number of stacked experts names an identity expert,
        whose output is the token's input, residual[t] += w h[t]."""
        self._routed(h, w, ids, weights, residual, shared, act, identity)

    def _shared_expert(self, h, shared, residual):
        w_gate_up, w_down, gate = shared
        y = torch.empty((h.shape[0], w_down.shape[1]), dtype=h.dtype, device=h.device)
        self.gate_up_swiglu(h, w_gate_up, y)
        self.scale_rows(y, gate)
        self.linear(y, w_down, residual, accumulate=True)

    def _routed(self, h, w, ids, weights, residual, shared, act=None, identity=False):
        from .state_ops import GLU_KINDS
        act_kind, act_limit, act_alpha = (0, 0.0, 0.0) if act is None else (GLU_KINDS[act[0]], float(act[1]), float(act[2]))
        _need(act_kind == 0 or shared is None, "routed_experts: a shared expert rides only with the silu activation")
        t, width = h.shape
        top = ids.shape[1]
        experts, ff = w["down"].shape[0], w["down"].shape[2]
        gate_up, interleaved = w["gate_up"], int(w["interleaved"])
        _need(gate_up.shape == (experts, 2 * ff, width) and w["down"].shape == (experts, width, ff),
              "routed_experts: expert shapes do not agree")
        _need(residual.dtype == torch.float32 and residual.stride(1) == 1 and tuple(residual.shape) == (t, width),
              "routed_experts: float32 residual")
        _need(h.stride(1) == 1, "routed_experts: rows must be contiguous")
        if (self.grouped_experts_from is not None and t * top >= self.grouped_experts_from
                and h.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16
                and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0
                and self.gated.ti_moe_grouped_supported(width, ff, experts)):
            pairs = t * top
            if (self.tcgen05_experts_from is not None and pairs >= self.tcgen05_experts_from and interleaved
                    and ff % 16 == 0 and width % 8 == 0):
                # every expert's pairs in whole tiles of 128 rows, the rows of h times their weights
                # gathered in that order, two grouped tcgen05 products (the first with SwiGLU in its
                # epilogue), and the pairs' rows added per token; with another activation the rows of h
                # are gathered as they are and the weights scale the pairs' rows as they are added
                max_rows = (pairs // 128 + experts) * 128
                ints = torch.empty(max_rows + pairs + max_rows // 128 + 1, dtype=torch.int32, device=h.device)
                row_pair, pos_of_pair = ints[:max_rows], ints[max_rows:max_rows + pairs]
                group_of_tile, tiles_m = ints[max_rows + pairs:-1], ints[-1:]
                g = self.gated
                self._ok(g.ti_moe_sort_padded(ids.data_ptr(), pairs, experts, max_rows, row_pair.data_ptr(),
                                              pos_of_pair.data_ptr(), group_of_tile.data_ptr(), tiles_m.data_ptr(),
                                              self._stream()), g)
                a = torch.empty((max_rows, width), dtype=torch.bfloat16, device=h.device)
                self._ok(g.ti_moe_gather_scaled(h.data_ptr(), h.stride(0), row_pair.data_ptr(), tiles_m.data_ptr(),
                                                weights.data_ptr() if act_kind == 0 else None, top, width, max_rows,
                                                a.data_ptr(), self._stream()), g)
                y = torch.empty((max_rows, ff), dtype=torch.bfloat16, device=h.device)
                self._ok(self.bf16.ti_gemm_tcgen05_grouped_glu(
                    a.data_ptr(), gate_up.data_ptr(), y.data_ptr(), max_rows, 2 * ff, width, width, width, ff,
                    experts, group_of_tile.data_ptr(), tiles_m.data_ptr(), act_kind, act_limit, act_alpha,
                    self.status.data_ptr(), self._stream()), self.bf16)
                out_rows = torch.empty((max_rows, width), dtype=torch.float32, device=h.device)
                self._ok(self.bf16.ti_gemm_tcgen05_grouped(
                    y.data_ptr(), w["down"].data_ptr(), out_rows.data_ptr(), None, max_rows, width, ff, ff, ff,
                    width, 0, 0, experts, group_of_tile.data_ptr(), tiles_m.data_ptr(), self.status.data_ptr(),
                    self._stream()), self.bf16)
                self._ok(g.ti_moe_combine_rows(out_rows.data_ptr(), pos_of_pair.data_ptr(), top, width, t,
                                               residual.data_ptr(), residual.stride(0),
                                               None if act_kind == 0 else weights.data_ptr(),
                                               ids.data_ptr() if identity else None, experts, weights.data_ptr(),
                                               h.data_ptr(), h.stride(0), self._stream()), g)
                if shared is not None:
                    self._shared_expert(h, shared, residual)
                return
            ints = torch.empty(pairs + 3 * (pairs // 64 + experts) + 1, dtype=torch.int32, device=h.device)
            y_sorted = torch.empty((pairs, ff), dtype=torch.bfloat16, device=h.device)
            out_rows = torch.empty((pairs, width), dtype=torch.float32, device=h.device)
            self._ok(self.gated.ti_moe_grouped(
                h.data_ptr(), h.stride(0), gate_up.data_ptr(), interleaved, w["down"].data_ptr(),
                ids.data_ptr(), weights.data_ptr(), t, top, experts, width, ff, ints.data_ptr(),
                ints[pairs:].data_ptr(), ints[ints.shape[0] - 1:].data_ptr(), y_sorted.data_ptr(),
                out_rows.data_ptr(), residual.data_ptr(), residual.stride(0), act_kind, act_limit, act_alpha,
                int(bool(identity)), self._stream()), self.gated)
            self.launches += 3
            if shared is not None:
                self._shared_expert(h, shared, residual)
            return
        # the CUDA-core kernels; a small shared expert of the experts' weight dtype rides along (two
        # launches instead of five).  A large one does not: these kernels fetch an expert's rows once
        # per pair, which for an expert that every token uses means once per token (measured at
        # batch 8: 5,784 -> 5,277 tok/s with a shared expert of 2,048 x 4,096 riding along)
        ride = (shared is not None and shared[0].dtype == gate_up.dtype and shared[1].dtype == gate_up.dtype
                and shared[0].is_contiguous() and shared[1].is_contiguous() and shared[2].dtype == torch.float32
                and shared[1].shape[1] * width <= self.shared_rides_to)
        y_sh = sgu = sdown = sgate = None
        s_ff = s_inter = 0
        if ride:
            sgu, sdown, sgate = shared
            s_ff, s_inter = sdown.shape[1], int(bool(getattr(sgu, "_ti_interleaved", False)))
            _need(tuple(sgu.shape) == (2 * s_ff, width) and tuple(sdown.shape) == (width, s_ff)
                  and sgate.shape[0] == t and sgate.is_contiguous(), "routed_experts: the shared expert's shapes")
            y_sh = torch.empty((t, s_ff), dtype=h.dtype, device=h.device)
        y = torch.empty((t, top, ff), dtype=h.dtype, device=h.device)
        self._ok(self.core.ti_moe_gate_up_simple(
            h.data_ptr(), _code(h, "routed_experts"), h.stride(0), gate_up.data_ptr(), interleaved,
            _code(gate_up, "routed_experts"), ids.data_ptr(), weights.data_ptr(), t, top, width, ff,
            y.data_ptr(), _ptr(sgu), s_inter, s_ff, _ptr(y_sh), act_kind, act_limit, act_alpha,
            experts if identity else 1 << 30, self._stream()))
        self._ok(self.core.ti_moe_down_simple(
            y.data_ptr(), _code(y, "routed_experts"), w["down"].data_ptr(), _code(w["down"], "routed_experts"),
            ids.data_ptr(), t, top, width, ff, residual.data_ptr(), residual.stride(0), _ptr(y_sh), _ptr(sdown),
            _ptr(sgate), s_ff, experts if identity else 1 << 30, h.data_ptr(), h.stride(0), weights.data_ptr(),
            self._stream()))
        if shared is not None and not ride:
            self._shared_expert(h, shared, residual)

    def scale_rows(self, y, factors):
        """y[r] *= factors[r] (float32 factors), in place."""
        _need(y.stride(1) == 1 and factors.dtype == torch.float32 and factors.shape[0] == y.shape[0]
              and factors.is_contiguous(), "scale_rows: one float32 factor per row")
        self._ok(self.core.ti_scale_rows(y.data_ptr(), _code(y, "scale_rows"), y.stride(0), factors.data_ptr(),
                                         y.shape[0], y.shape[1], self._stream()))

    # ---- sampling ------------------------------------------------------------------------
    def argmax(self, logits, out):
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "argmax: float32 logits")
        _need(out.dtype == torch.int32 and out.shape[0] == logits.shape[0], "argmax: int32 out")
        rows, vocab = logits.shape
        if vocab >= 16384:                 # wide rows: many blocks per row, then one pick
            part_v = torch.empty((rows, 64), dtype=torch.float32, device=logits.device)
            part_i = torch.empty((rows, 64), dtype=torch.int32, device=logits.device)
            self._ok(self.core.ti_argmax_sliced(logits.data_ptr(), rows, vocab, part_v.data_ptr(),
                                                part_i.data_ptr(), out.data_ptr(), self._stream()))
            return
        self._ok(self.core.ti_argmax(logits.data_ptr(), rows, vocab, out.data_ptr(), self._stream()))

    def sample(self, logits, temperature, top_k, top_p, uniform, out):
        rows = logits.shape[0]
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: float32 logits")
        for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                            ("top_p", top_p, torch.float32), ("uniform", uniform, torch.float32),
                            ("out", out, torch.int32)):
            _need(t.dtype == dt and t.shape[0] == rows and t.is_contiguous(),
                  f"sample: {name} must be {dt} with one value per row")
        self._ok(self.core.ti_sample(logits.data_ptr(), rows, logits.shape[1],
                                     temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                                     uniform.data_ptr(), out.data_ptr(), self._stream()))


CudaOps._ROTATIONS = {"neox": CudaOps._rotate_builtin, "none": CudaOps._rotate_builtin}


def _flush_first(fn):
    """Other operations launch what ``linear(..., may_defer=True)`` has held back before they run."""
    import functools

    @functools.wraps(fn)
    def wrapper(self, *args, **kwargs):
        if self._pending is not None or self._pending_runs is not None:
            self.flush()
        return fn(self, *args, **kwargs)
    return wrapper


for _name, _fn in list(vars(MixerOps).items()) + list(vars(StateOps).items()) + list(vars(CudaOps).items()):
    if (isinstance(_fn, type(_flush_first)) and not _name.startswith("_")
            and _name not in ("flush", "linear", "rmsnorm", "swiglu_ffn")):
        setattr(CudaOps, _name, _flush_first(_fn))
del _name, _fn
