"""Bindings of the kernels in ``csrc/attn_options.cu`` and ``csrc/wkv.cu`` (library ``mixers``):
attention with optional parts (chunk or window mask, a score factor per head, a cap on the score,
a sink in the softmax, an output gate per head or per element, keys and values read from one
shared row), the kernels that prepare its heads, and a recurrent mixer with a matrix state.

``CudaOps`` inherits these methods; the library is built when one of them is first called, so
a model without such mixers never compiles it.

qk_rownorm_rope_store(proj, ...)     norm over the whole query row and the whole key row, turn
                                     of neighbouring pairs, keys/values into pages, queries out
latent_prepare(proj, ...)            normed latent + turned key part as one cached row; plain
                                     and turned query parts out
qkv_turn_store(proj, ...)            no norm: queries and keys turned, values turned by frequencies of
                                     their own, keys/values into pages, queries out
slice_rmsnorm(x, weight, eps, out)   RMS norm of a column slice of a product
turn_rows(x, step, rotation, ...)    finished rows' heads turned by plus or minus their position, times
                                     sigmoid(gate)
head_project(x, w, out)              out[t, h] = x[t, h] @ w[h]
attention_options(q, step, cache, out, ...)
token_shift_mix(h, mu, step, state, out)
wkv_recurrence(r, k, v, g, a, ..., step, state, out)
tanh_rows(x, out) / xielu_rows(x, ap, aq, out)
"""
from __future__ import annotations

import ctypes

import torch

from .build import load_library

_CODE = {torch.float32: 0, torch.bfloat16: 1}
_vp, _i, _f, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def _ptr(t):
    return None if t is None else t.data_ptr()


class MixerOps:
    _mixers = None
    _mixers_tc = None
    use_tc_attention_options = True        # tensor-core kernel of the attention with options (bfloat16)

    @property
    def _row_tile_tokens(self) -> set:
        found = self.__dict__.get("_row_tile_set")
        if found is None:
            found = self.__dict__["_row_tile_set"] = set()
        return found

    def want_row_tiles(self, num_heads: int, num_kv_heads: int) -> None:
        """A mixer says, when it gets its weights, that it will call ``attention_options`` with these
        head counts: every step then brings the tile list that the tensor-core kernel walks
        (``step_lists``); without it the calls run on the CUDA-core kernel."""
        self._row_tile_tokens.add(64 // self._group_rows(num_heads, num_kv_heads))

    @staticmethod
    def _group_rows(num_heads: int, num_kv_heads: int) -> int:
        gp = 1
        while gp < num_heads // num_kv_heads and gp < 64:
            gp *= 2
        return gp

    @property
    def mixers_tc(self):
        if self._mixers_tc is None:
            b = load_library("bf16_mixers")
            b.ti_last_error.restype = ctypes.c_char_p
            b.ti_attn_options_tc_supported.argtypes = [_i, _i, _i, _i]
            b.ti_attn_options_tc_group_rows.argtypes = [_i, _i]
            b.ti_head_project_tc_supported.argtypes = [_i, _i, _i, _i]
            b.ti_head_project_tc.argtypes = [_vp, _i, _i, _vp, _i, _i, _vp, _i, _i, _i, _i, _vp]
            b.ti_attn_options_tc.argtypes = [_vp, _vp, _i, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i,
                                             _f, _f, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _vp]
            self._mixers_tc = b
        return self._mixers_tc

    @property
    def mixers(self):
        if self._mixers is None:
            b = load_library("mixers")
            b.ti_last_error.restype = ctypes.c_char_p
            b.ti_qk_rownorm_rope_store.argtypes = [_vp, _i, _vp, _vp, _f, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i,
                                                   _i, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp]
            b.ti_latent_prepare.argtypes = [_vp, _i, _vp, _i, _vp, _f, _vp, _f, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i,
                                            _i, _i, _i, _vp, _vp, _i, _vp, _vp]
            b.ti_qkv_turn_store.argtypes = [_vp, _i, _vp, _i, _i, _f, _vp, _i, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i,
                                            _i, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp]
            b.ti_slice_rmsnorm.argtypes = [_vp, _i, _i, _i, _vp, _f, _vp, _i, _vp]
            b.ti_turn_rows.argtypes = [_vp, _i, _vp, _vp, _i, _i, _f, _vp, _i, _i, _i, _i, _vp, _vp]
            b.ti_head_project.argtypes = [_vp, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _vp]
            b.ti_attention_options.argtypes = [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i,
                                               _i, _i, _i, _f, _f, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp]
            b.ti_token_shift_mix.argtypes = [_vp, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _ll, _ll, _vp, _vp]
            b.ti_wkv_recurrence.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _f, _vp, _i, _i, _vp, _vp,
                                            _vp, _ll, _ll, _i, _i, _i, _i, _i, _vp, _vp, _vp]
            b.ti_tanh_rows.argtypes = [_vp, _ll, _vp, _i, _vp]
            b.ti_xielu_rows.argtypes = [_vp, _ll, _f, _f, _vp, _i, _vp]
            self._mixers = b
        return self._mixers

    def _mx(self, rc: int) -> None:
        self._ok(rc, self.mixers)

    @staticmethod
    def _must(cond: bool, msg: str) -> None:
        if not cond:
            from .cuda_ops import KernelError
            raise KernelError(msg)

    # ---- preparing heads ---------------------------------------------------------------------
    def qk_rownorm_rope_store(self, proj, q_weight, k_weight, eps, rotation, step, cache, q_out,
                              num_heads, num_kv_heads, dk, dv, per_head=False):
        """From the float32 product ``proj`` (columns: queries, keys, values, then anything else):
        RMS norm over the whole query row and over the whole key row (weights of that length, or
        None), rotation of the first ``rotation.rotary_dim`` elements of every head in neighbouring
        pairs (kind ``interleaved``) or none, keys and values into the token's page (if the cache
        slot is written), queries into ``q_out``.  ``per_head``: every query head and every key
        head is normed by itself (RMS over ``dk``) with a weight of ``dk`` elements that all heads
        share."""
        t = proj.shape[0]
        pages, bt = cache.pages, cache.block_table
        nq, nk, nv = num_heads * dk, num_kv_heads * dk, num_kv_heads * dv
        self._must(rotation.kind in ("interleaved", "none"),
                   f"qk_rownorm_rope_store turns neighbouring pairs; rotation kind {rotation.kind!r} is not that")
        rot = int(rotation.rotary_dim)
        self._must(getattr(rotation, "scale", 1.0) == 1.0, "qk_rownorm_rope_store: a pure turn only (no factor on sine and cosine)")
        self._must(proj.dtype == torch.float32 and proj.stride(1) == 1
                   and proj.shape[1] >= nq + (nk + nv if cache.writes else 0),
                   "qk_rownorm_rope_store: the product must be float32 and hold all heads")
        for w, n in ((q_weight, dk if per_head else nq), (k_weight, dk if per_head else nk)):
            self._must(w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.shape[0] == n),
                       "qk_rownorm_rope_store: a norm weight must be float32, one value per column")
        self._must(rot == 0 or (rotation.inv_freq is not None and rotation.inv_freq.dtype == torch.float32
                                and rotation.inv_freq.shape[0] >= rot // 2),
                   "qk_rownorm_rope_store: the rotation needs rotary_dim/2 float32 frequencies")
        self._must(pages.is_contiguous() and pages[0].numel() == num_kv_heads * cache.page_size * (dk + dv),
                   "qk_rownorm_rope_store: page layout")
        self._must(bt.dtype == torch.int32 and bt.stride(1) == 1, "qk_rownorm_rope_store: block table int32")
        self._must(q_out.is_contiguous() and tuple(q_out.shape) == (t, nq), "qk_rownorm_rope_store: q_out")
        self._mx(self.mixers.ti_qk_rownorm_rope_store(
            proj.data_ptr(), proj.stride(0), _ptr(q_weight), _ptr(k_weight), float(eps),
            _ptr(rotation.inv_freq) if rot else None, rot, step.positions.data_ptr(), step.req_of_tok.data_ptr(),
            bt.data_ptr(), bt.stride(0), pages.data_ptr(), _CODE[pages.dtype], pages.shape[0], cache.page_size,
            int(bool(cache.writes)), t, num_heads, num_kv_heads, dk, dv, int(bool(per_head)), q_out.data_ptr(),
            _CODE[q_out.dtype], self.status.data_ptr(), self._stream()))

    def latent_prepare(self, proj, latent_weight, eps, rotation, step, cache, q_plain, q_full,
                       num_heads, dk, dr, rank, q_proj=None):
        """From the float32 product ``proj`` (columns: per head ``dk`` plain and ``dr`` rotated
        query elements, then the latent of ``rank`` elements and one rotated key part of ``dr``):
        the latent, normed (weight or None), and the turned key part go into the token's page as one
        row of ``rank + dr``; ``q_plain`` ``[T, heads * dk]`` gets the plain query parts and
        ``q_full[:, h, rank:]`` (``[T, heads, rank + dr]``) the turned ones.  With ``q_proj`` the
        query heads are its columns and ``proj`` starts with the latent.  The sines and cosines of
        both turned parts are multiplied by ``rotation.scale``."""
        t = proj.shape[0]
        pages, bt = cache.pages, cache.block_table
        nq = num_heads * (dk + dr)
        self._must(dr == 0 or (rotation.kind == "interleaved" and rotation.rotary_dim == dr),
                   "latent_prepare turns the whole rotated part in neighbouring pairs")
        if q_proj is None:
            q_proj, proj = proj, proj[:, nq:]
        self._must(proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= rank + dr
                   and q_proj.dtype == torch.float32 and q_proj.stride(1) == 1 and q_proj.shape[1] >= nq
                   and q_proj.shape[0] == t,
                   "latent_prepare: the products must be float32 and hold queries, latent and key part")
        self._must(latent_weight is None or (latent_weight.dtype == torch.float32 and latent_weight.shape[0] == rank),
                   "latent_prepare: the latent's norm weight must be float32")
        self._must(pages.is_contiguous() and pages[0].numel() == cache.page_size * (rank + dr),
                   "latent_prepare: a page holds one row of rank + dr per token")
        self._must(bt.dtype == torch.int32 and bt.stride(1) == 1, "latent_prepare: block table int32")
        self._must(q_plain.is_contiguous() and q_full.is_contiguous() and q_plain.dtype == q_full.dtype
                   and tuple(q_plain.shape) == (t, num_heads * dk)
                   and q_full.numel() == t * num_heads * (rank + dr), "latent_prepare: query outputs")
        self._must(bool(cache.writes), "latent_prepare writes the cache slot")
        self._mx(self.mixers.ti_latent_prepare(
            q_proj.data_ptr(), q_proj.stride(0), proj.data_ptr(), proj.stride(0), _ptr(latent_weight), float(eps),
            _ptr(rotation.inv_freq) if dr else None, float(getattr(rotation, "scale", 1.0)),
            step.positions.data_ptr(), step.req_of_tok.data_ptr(),
            bt.data_ptr(), bt.stride(0), pages.data_ptr(), _CODE[pages.dtype], pages.shape[0], cache.page_size,
            t, num_heads, dk, dr, rank, q_plain.data_ptr(), q_full.data_ptr(), _CODE[q_plain.dtype],
            self.status.data_ptr(), self._stream()))

    def slice_rmsnorm(self, x, weight, eps, out):
        """``out = x / sqrt(mean(x^2) + eps) * weight`` per row, for float32 rows ``x`` that may be a
        column slice of a wider product (any row stride); ``weight`` float32 per element or None."""
        t, n = x.shape
        self._must(x.dtype == torch.float32 and x.stride(1) == 1 and out.is_contiguous() and tuple(out.shape) == (t, n)
                   and (weight is None or (weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == n)),
                   "slice_rmsnorm: float32 rows, a float32 weight per element, contiguous rows out")
        self._mx(self.mixers.ti_slice_rmsnorm(x.data_ptr(), x.stride(0), t, n, _ptr(weight), float(eps), out.data_ptr(),
                                              _CODE[out.dtype], self._stream()))

    _LAYOUTS = {"interleaved": 0, "neox": 1}

    def qkv_turn_store(self, proj, rotation, v_rotation, step, cache, q_out, num_heads, num_kv_heads, dk, dv):
        """From the float32 rows ``proj`` (columns: queries, keys, values): no norm; the first
        ``rotation.rotary_dim`` elements of every query and key head are turned by the token's
        position (kind ``interleaved``: neighbouring pairs; ``neox``: element ``i`` with ``i +
        rotary_dim / 2``; ``none``), the first ``v_rotation.rotary_dim`` elements of every value
        head by ``v_rotation`` (or None: values as they are); keys and values go into the token's
        page (if the cache slot is written), queries into ``q_out``."""
        t = proj.shape[0]
        pages, bt = cache.pages, cache.block_table
        nq, nk, nv = num_heads * dk, num_kv_heads * dk, num_kv_heads * dv
        rots = []
        for what, r, size in (("heads", rotation, dk), ("values", v_rotation, dv)):
            n = 0 if r is None or r.kind == "none" else int(r.rotary_dim)
            self._must(n == 0 or (r.kind in self._LAYOUTS and r.inv_freq is not None and r.inv_freq.dtype == torch.float32
                                  and r.inv_freq.shape[0] >= n // 2 and n <= size),
                       f"qkv_turn_store: the rotation of the {what} needs a known pairing and rotary_dim/2 float32 frequencies")
            rots.append((n, self._LAYOUTS.get(r.kind, 0) if n else 0, _ptr(r.inv_freq) if n else None,
                         float(getattr(r, "scale", 1.0)) if n else 1.0))
        self._must(rots[1][3] == 1.0, "qkv_turn_store: values are turned without a factor")
        self._must(proj.dtype == torch.float32 and proj.stride(1) == 1
                   and proj.shape[1] >= nq + (nk + nv if cache.writes else 0),
                   "qkv_turn_store: the rows must be float32 and hold all heads")
        self._must(pages.is_contiguous() and pages[0].numel() == num_kv_heads * cache.page_size * (dk + dv),
                   "qkv_turn_store: page layout")
        self._must(bt.dtype == torch.int32 and bt.stride(1) == 1, "qkv_turn_store: block table int32")
        self._must(q_out.is_contiguous() and tuple(q_out.shape) == (t, nq), "qkv_turn_store: q_out")
        self._mx(self.mixers.ti_qkv_turn_store(
            proj.data_ptr(), proj.stride(0), rots[0][2], rots[0][0], rots[0][1], rots[0][3], rots[1][2], rots[1][0],
            rots[1][1], step.positions.data_ptr(), step.req_of_tok.data_ptr(), bt.data_ptr(), bt.stride(0),
            pages.data_ptr(), _CODE[pages.dtype], pages.shape[0], cache.page_size, int(bool(cache.writes)), t,
            num_heads, num_kv_heads, dk, dv, q_out.data_ptr(), _CODE[q_out.dtype], self.status.data_ptr(),
            self._stream()))

    def turn_rows(self, x, step, rotation, num_heads, n, back=False, gate=None, out=None):
        """``out[t, h, :]`` is head ``h`` of row ``t`` of ``x`` (``[T, heads * n]``) with its first
        ``rotation.rotary_dim`` elements turned by the token's position, or, ``back``, by minus the
        position; then times ``sigmoid(gate)`` (float32 ``[T, heads * n]``) if given.  ``out`` None:
        in place."""
        t = x.shape[0]
        out = x if out is None else out
        rot = 0 if rotation is None or rotation.kind == "none" else int(rotation.rotary_dim)
        self._must(x.is_contiguous() and out.is_contiguous() and x.dtype == out.dtype
                   and tuple(x.shape) == tuple(out.shape) == (t, num_heads * n), "turn_rows: contiguous [T, heads * n] rows")
        self._must(rot == 0 or (rotation.kind in self._LAYOUTS and rotation.inv_freq is not None
                                and rotation.inv_freq.dtype == torch.float32 and rotation.inv_freq.shape[0] >= rot // 2),
                   "turn_rows: the rotation needs a known pairing and rotary_dim/2 float32 frequencies")
        self._must(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1
                                    and tuple(gate.shape) == (t, num_heads * n)), "turn_rows: a float32 gate per element")
        self._mx(self.mixers.ti_turn_rows(
            x.data_ptr(), _CODE[x.dtype], step.positions.data_ptr(), _ptr(rotation.inv_freq) if rot else None, rot,
            self._LAYOUTS.get(rotation.kind, 0) if rot else 0, -1.0 if back else 1.0, _ptr(gate),
            gate.stride(0) if gate is not None else 0, t, num_heads, n, out.data_ptr(), self._stream()))

    def head_project(self, x, w, out):
        """``out[t, h, :] = x[t, h, :] @ w[h]`` for ``x [T, heads, n_in]``, ``w [heads, n_in, n_out]``
        and ``out [T, heads, n_out]``; ``x`` and ``out`` may be views with strides over tokens and
        heads (their last axis contiguous)."""
        t, heads, n_in = x.shape
        n_out = w.shape[2]
        self._must(tuple(w.shape) == (heads, n_in, n_out) and w.is_contiguous()
                   and tuple(out.shape) == (t, heads, n_out), "head_project: shapes do not agree")
        self._must(x.stride(2) == 1 and out.stride(2) == 1 and x.dtype == out.dtype,
                   "head_project: contiguous last axes and one dtype for input and output")
        if (t > 64 and x.dtype == w.dtype == torch.bfloat16 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and self.mixers_tc.ti_head_project_tc_supported(n_in, n_out, x.stride(0), x.stride(1))):
            # many tokens: on the tensor cores
            self._ok(self.mixers_tc.ti_head_project_tc(
                x.data_ptr(), x.stride(0), x.stride(1), w.data_ptr(), n_in, n_out, out.data_ptr(), out.stride(0),
                out.stride(1), t, heads, self._stream()), self.mixers_tc)
            return
        self._mx(self.mixers.ti_head_project(
            x.data_ptr(), _CODE[x.dtype], x.stride(0), x.stride(1), w.data_ptr(), _CODE[w.dtype], n_in, n_out,
            out.data_ptr(), _CODE[out.dtype], out.stride(0), out.stride(1), t, heads, self._stream()))

    # ---- attention ---------------------------------------------------------------------------
    def attention_options(self, q, step, cache, out, num_heads, num_kv_heads, dk, dv, scale, *,
                          window=None, chunk=None, softcap=None, head_scale=None, sink=None, gate=None,
                          gate_per_head=False, shared_rows=False):
        """Causal attention over the pages of each token's request.  Token ``i`` sees key ``j <= i``
        with ``i - j < window`` (if a window is given) and ``j >= (i // chunk) * chunk`` (if a chunk
        is given).  ``score = (q . k) * scale [* head_scale[h]]``, then ``softcap * tanh(score /
        softcap)`` if given; the softmax's denominator also counts ``exp(sink[h])`` if given; the
        output is multiplied by ``sigmoid(gate)``: ``gate`` float32 ``[T, heads]`` (per head) or
        ``[T, heads * dv]``.  ``shared_rows``: a page holds one row of ``dk`` elements per token
        and kv head, whose first ``dv`` elements are the value."""
        pages, bt = cache.pages, cache.block_table
        t = q.shape[0]
        self._must(q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype
                   and q.numel() == t * num_heads * dk and out.numel() == t * num_heads * dv,
                   "attention_options: q and out must be contiguous [T, heads * size] of one dtype")
        per_page = num_kv_heads * cache.page_size * (dk if shared_rows else dk + dv)
        self._must(pages.is_contiguous() and pages[0].numel() == per_page, "attention_options: page layout")
        for name, v in (("head_scale", head_scale), ("sink", sink)):
            self._must(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.shape[0] == num_heads),
                       f"attention_options: {name} must be float32, one value per head")
        self._must(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == t
                                    and gate.shape[1] == (num_heads if gate_per_head else num_heads * dv)),
                   "attention_options: the gate must be float32 [T, heads] or [T, heads * dv]")
        gp = self._group_rows(num_heads, num_kv_heads)
        tiles = getattr(step, "lists", {}).get(f"row_tiles_{64 // gp}")
        if (self.use_tc_attention_options and tiles is not None and 0 < tiles.shape[0] <= 65535 and q.dtype == torch.bfloat16
                and pages.dtype == torch.bfloat16 and q.data_ptr() % 16 == 0 and out.data_ptr() % 4 == 0
                and pages.data_ptr() % 16 == 0
                and self.mixers_tc.ti_attn_options_tc_supported(dk, dv, cache.page_size, int(bool(shared_rows)))
                and self.mixers_tc.ti_attn_options_tc_group_rows(num_heads, num_kv_heads) == gp):
            # a step of single tokens has few blocks: the keys of a row in runs, a block each; the
            # count depends on the step's shape and the model's bounds alone
            nsplit, part_o, part_ml = 1, None, None
            slices = dv // (128 if dv % 128 == 0 else 64 if dv % 64 == 0 else 32 if dv % 32 == 0 else 16)
            single = getattr(step, "max_q_len", 0) == 1
            # single tokens of few heads: the warps of a block share the rows and split the keys (1) or,
            # over shared rows, the slices of the value columns (2)
            mode = 0 if not single else 2 if (shared_rows and 1 < slices <= 4) else 1 if gp <= 16 else 0
            if mode == 0 and shared_rows and dv % 256 == 0:
                slices = dv // 256                    # prompt portions over shared rows: 256 columns a block
            head_blocks = -(-(num_heads // num_kv_heads) // (min(gp, 16) if mode == 2 else gp))
            blocks = tiles.shape[0] * num_kv_heads * head_blocks * (1 if mode == 2 else slices)
            if single and blocks < 2 * self.num_sms:
                most = step.max_position or step.max_ctx_len
                for bound in (window, chunk):
                    if bound:
                        most = min(most, int(bound))
                nsplit = max(1, min(2 * self.num_sms // blocks, -(-most // 64) // 2, 64))
            if nsplit > 1:
                part_o = torch.empty((t, num_heads, nsplit, dv), dtype=torch.float32, device=q.device)
                part_ml = torch.empty((t, num_heads, nsplit, 2), dtype=torch.float32, device=q.device)
                self.launches += 1
            self._ok(self.mixers_tc.ti_attn_options_tc(
                q.data_ptr(), tiles.data_ptr(), tiles.shape[0], t, step.positions.data_ptr(), bt.data_ptr(),
                bt.stride(0), pages.data_ptr(), pages.shape[0], cache.page_size, num_heads, num_kv_heads, dk, dv,
                int(bool(shared_rows)), int(window or 0), int(chunk or 0), float(scale), float(softcap or 0.0),
                _ptr(head_scale), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0,
                int(bool(gate_per_head)), nsplit, _ptr(part_o), _ptr(part_ml),
                mode, out.data_ptr(),
                self.status.data_ptr(), self._stream()), self.mixers_tc)
            return
        self._mx(self.mixers.ti_attention_options(
            q.data_ptr(), _CODE[q.dtype], None, step.positions.data_ptr(), step.req_of_tok.data_ptr(),
            bt.data_ptr(), bt.stride(0), pages.data_ptr(), _CODE[pages.dtype], pages.shape[0], cache.page_size,
            t, num_heads, num_kv_heads, dk, dv, int(bool(shared_rows)), int(window or 0), int(chunk or 0),
            float(scale), float(softcap or 0.0), _ptr(head_scale), _ptr(sink), _ptr(gate),
            gate.stride(0) if gate is not None else 0, int(bool(gate_per_head)), out.data_ptr(),
            self.status.data_ptr(), self._stream()))

    # ---- the recurrent mixer -------------------------------------------------------------------
    def token_shift_mix(self, h, mu, step, state, prev_offset, out):
        """``out[s, t] = h[t] + (h'[t] - h[t]) * mu[s]`` with ``h'[t]`` the row of the token before
        ``t`` in its request: the row above, or for a request's first token of this step the row
        kept in its state slot at ``prev_offset`` (``state.state`` is float32 ``[slots, n]``)."""
        t, width = h.shape
        n_mix = mu.shape[0]
        st = state.state
        self._must(h.is_contiguous() and out.is_contiguous() and out.dtype == h.dtype
                   and tuple(out.shape) == (n_mix, t, width), "token_shift_mix: out must be [mixes, T, width]")
        self._must(mu.dtype == torch.float32 and mu.is_contiguous() and mu.shape[1] == width,
                   "token_shift_mix: mu must be float32 [mixes, width]")
        self._must(st.dtype == torch.float32 and st.is_contiguous() and st[0].numel() >= prev_offset + width,
                   "token_shift_mix: the state must be float32 and hold the kept row")
        self._mx(self.mixers.ti_token_shift_mix(
            h.data_ptr(), _CODE[h.dtype], mu.data_ptr(), n_mix, width, t, step.req_of_tok.data_ptr(),
            step.cu_q.data_ptr(), state.slots.data_ptr(), st.data_ptr(), st[0].numel(), int(prev_offset),
            out.data_ptr(), self._stream()))

    def wkv_recurrence(self, r, k, v, g, a, w0, u, norm_weight, eps, h, step, state, prev_offset, out,
                       num_heads, d):
        """Per request and head, over the request's tokens in order, with ``S`` the head's state
        ``[d, d]`` at the start of the slot: ``decay = exp(-exp(a + w0))``, ``o = (S + diag(u) k
        v^T)^T r``, ``S <- diag(decay) S + k v^T``; ``out = o / rms(o) * norm_weight * silu(g)``.
        ``r, k, v, g, a`` are float32 ``[T, heads * d]`` views of one row stride.  The state slot
        gets the new ``S`` and, at ``prev_offset``, the request's last row of ``h``."""
        t = h.shape[0]
        n = num_heads * d
        st = state.state
        for x in (r, k, v, g, a):
            self._must(x.dtype == torch.float32 and x.stride(1) == 1 and tuple(x.shape) == (t, n)
                       and x.stride(0) == r.stride(0), "wkv_recurrence: float32 [T, heads * d] inputs of one stride")
        for x in (w0, u, norm_weight):
            self._must(x.dtype == torch.float32 and x.is_contiguous() and x.numel() == n,
                       "wkv_recurrence: float32 vectors of heads * d")
        self._must(st.dtype == torch.float32 and st.is_contiguous() and prev_offset >= num_heads * d * d
                   and st[0].numel() >= prev_offset + h.shape[1], "wkv_recurrence: the state slot is too small")
        self._must(h.is_contiguous() and out.is_contiguous() and out.dtype == h.dtype and tuple(out.shape) == (t, n),
                   "wkv_recurrence: out must be [T, heads * d] in the activation dtype")
        self._must(bool(state.writes), "wkv_recurrence writes its state")
        # long portions of few requests leave most SMs without a head: a head's state columns are then
        # cut over four blocks, and a second launch takes the norm and the gate (a rule of the step's
        # shape alone)
        split = 4 if (step.max_q_len >= 64 and step.num_requests * num_heads * 2 <= self.num_sms) else 1
        o_raw = torch.empty((t, n), dtype=torch.float32, device=h.device) if split > 1 else None
        if split > 1:
            self.launches += 1
        self._mx(self.mixers.ti_wkv_recurrence(
            r.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), a.data_ptr(), r.stride(0), w0.data_ptr(),
            u.data_ptr(), norm_weight.data_ptr(), float(eps), h.data_ptr(), _CODE[h.dtype], h.shape[1],
            step.cu_q.data_ptr(), state.slots.data_ptr(), st.data_ptr(), st[0].numel(), int(prev_offset),
            step.num_requests, t, num_heads, d, split, _ptr(o_raw), out.data_ptr(), self._stream()))

    # ---- activations ---------------------------------------------------------------------------
    def tanh_rows(self, x, out):
        self._must(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
                   and out.shape == x.shape, "tanh_rows: contiguous float32 in, same shape out")
        self._mx(self.mixers.ti_tanh_rows(x.data_ptr(), x.numel(), out.data_ptr(), _CODE[out.dtype], self._stream()))

    def xielu_rows(self, x, ap, aq, out):
        """``out = ap z^2 + z/2`` where ``z > 0``, ``aq (exp(z) - 1 - z) + z/2`` elsewhere."""
        self._must(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
                   and out.shape == x.shape, "xielu_rows: contiguous float32 in, same shape out")
        self._mx(self.mixers.ti_xielu_rows(x.data_ptr(), x.numel(), float(ap), float(aq), out.data_ptr(),
                                           _CODE[out.dtype], self._stream()))
