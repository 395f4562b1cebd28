"""Bindings of the kernels in ``csrc/matrix_state.cu`` (library ``state``) and
``csrc/state_rows.cu`` (library ``rows``): recurrent mixers with a float32 matrix state per head, short causal convolutions
over time with their kept inputs, norms in groups, the depth-weighted mix of layer outputs, and
gated activations with clamps.

``CudaOps`` inherits these methods; each library is built when one of its kernels is first called, so
a model without a recurrence never compiles ``state``, and one without any of these parts neither.

causal_conv(x, w, step, state, offset, out, add_input, silu)   y = [x +] conv(x) [silu], rows before a portion from the state
conv_tail_store(x, taps, step, state, offset)                  the state's kept inputs renewed after a step
group_norm(x, w, eps, groups, out | residual, rows)            RMS norm in equal consecutive parts of a row
tanh_norm(x, alpha, w, b, out | residual, rows)                tanh(alpha x) w + b, the norm without mean or variance
tanh_norm_pair(y, ..., residual, ..., out)                     residual += norm1(y); out = norm2(residual)
cap_rows(x, cap)                                               x = cap tanh(x / cap), in place
add_row(x, row)                                                x[t] += row
depth_mix(x, hist, index, weights)                             hist[index] = x; x = sum_j weights[j] hist[j]
add_scaled(dst, a, sa, b, sb)                                  dst += sa a + sb b
glu_rows(gu, interleaved, kind, limit, alpha, out)             out = act(gate, up)
matrix_state(mode, ...)                                        the gated delta rule / the gated sum of outer products
"""
from __future__ import annotations

import ctypes

import torch

from .build import load_library

_CODE = {torch.float32: 0, torch.bfloat16: 1}
_vp, _i, _f, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

GLU_KINDS = {"silu": 0, "clamped": 1}
STATE_MODES = {"delta": 0, "gated_sum": 1}
GATE_ACTS = {"silu": 0, "sigmoid": 1}


def _ptr(t):
    return None if t is None else t.data_ptr()


def matrix_state_floats(mode: str, heads: int, dk: int, dv: int) -> int:
    """Floats of state a request keeps for one layer of the recurrence ``mode``."""
    return heads * dk * (dv + 1) + heads if mode == "gated_sum" else heads * dk * dv


class StateOps:
    _state_lib = None
    cut_state_columns = True          # long portions of few requests: a head's columns over several blocks

    _rows_lib = None

    @property
    def state_lib(self):
        if self._state_lib is None:
            b = load_library("state")
            b.ti_last_error.restype = ctypes.c_char_p
            b.ti_matrix_state.argtypes = [_i, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp, _i, _vp, _vp, _f, _vp, _i, _i,
                                          _vp, _i, _f, _vp, _vp, _i, _i, _vp, _ll, _i, _i, _i, _i, _i, _vp, _i, _vp,
                                          _vp, _vp]
            self._state_lib = b
        return self._state_lib

    @property
    def rows_lib(self):
        if self._rows_lib is None:
            b = load_library("rows")
            b.ti_last_error.restype = ctypes.c_char_p
            b.ti_causal_conv_rows.argtypes = [_vp, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _vp,
                                              _i, _i, _vp]
            b.ti_conv_tail_store.argtypes = [_vp, _i, _i, _i, _vp, _vp, _i, _vp, _ll, _ll, _vp]
            b.ti_group_norm_rows.argtypes = [_vp, _vp, _vp, _i, _i, _i, _f, _vp, _i, _vp, _i, _vp]
            b.ti_tanh_norm_rows.argtypes = [_vp, _vp, _i, _i, _f, _vp, _vp, _vp, _i, _vp, _i, _vp]
            b.ti_tanh_norm_pair.argtypes = [_vp, _i, _i, _f, _vp, _vp, _vp, _i, _f, _vp, _vp, _vp, _i, _vp]
            b.ti_cap_rows.argtypes = [_vp, _ll, _f, _vp]
            b.ti_add_row.argtypes = [_vp, _i, _vp, _i, _i, _vp]
            b.ti_depth_mix.argtypes = [_vp, _vp, _ll, _i, _vp, _vp]
            b.ti_add_scaled.argtypes = [_vp, _i, _vp, _f, _vp, _f, _i, _i, _vp]
            b.ti_glu_rows.argtypes = [_vp, _i, _i, _i, _i, _f, _f, _vp, _i, _vp]
            self._rows_lib = b
        return self._rows_lib

    def _rw(self, rc: int) -> None:
        self._ok(rc, self.rows_lib)

    def _st(self, rc: int) -> None:
        self._ok(rc, self.state_lib)

    @staticmethod
    def _want(cond: bool, msg: str) -> None:
        if not cond:
            from .cuda_ops import KernelError
            raise KernelError(msg)

    # ---- short convolutions over time ----------------------------------------------------------
    def causal_conv(self, x, w, step, state, state_offset, out, add_input=False, silu=False, renew=False):
        """``out[t, c] = [x[t, c] +] sum_j w[c, j] x[t - taps + 1 + j, c]``, then silu if asked, over
        float32 rows ``x`` (a column slice is fine).  Rows before a request's portion come from
        ``state`` (a ``StateView``: per slot ``[taps - 1, channels]`` floats from ``state_offset``
        on, the newest row last).  ``w`` None: the rows are converted (and nothing else).
        ``renew``: the kept rows become the requests' last inputs after this step, in the same
        launch where every request brings one token, else by ``conv_tail_store`` behind it."""
        t, c = x.shape
        taps = 0 if w is None else w.shape[1]
        self._want(x.dtype == torch.float32 and x.stride(1) == 1 and out.stride(1) == 1
                   and tuple(out.shape) == (t, c), "causal_conv: float32 rows in, rows of the same shape out")
        self._want(w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.shape[0] == c),
                   "causal_conv: float32 weights [channels, taps]")
        st = None if state is None else state.state
        self._want(taps <= 1 or (st is not None and st.dtype == torch.float32
                                 and st[0].numel() >= state_offset + (taps - 1) * c),
                   "causal_conv: the state must hold taps - 1 float32 rows")
        renew = bool(renew) and taps > 1 and state.writes
        in_place = renew and step.max_q_len == 1 and step.num_requests == t
        self._rw(self.rows_lib.ti_causal_conv_rows(
            x.data_ptr(), x.stride(0), _ptr(w), taps, c, t, step.req_of_tok.data_ptr(), step.cu_q.data_ptr(),
            _ptr(state.slots) if state is not None else None, _ptr(st), st.stride(0) if st is not None else 0,
            int(state_offset), int(bool(add_input)), int(bool(silu)), int(in_place), out.data_ptr(), _CODE[out.dtype],
            out.stride(0), self._stream()))
        if renew and not in_place:
            self.conv_tail_store(x, taps, step, state, state_offset)

    def conv_tail_store(self, x, taps, step, state, state_offset):
        """The state's ``taps - 1`` kept rows of every request become its last inputs after this
        step.  Launched behind every reader of the old rows."""
        if taps <= 1 or not state.writes:
            return
        c = x.shape[1]
        st = state.state
        self._want(x.dtype == torch.float32 and x.stride(1) == 1, "conv_tail_store: float32 rows")
        self._rw(self.rows_lib.ti_conv_tail_store(
            x.data_ptr(), x.stride(0), int(taps), c, step.cu_q.data_ptr(), state.slots.data_ptr(),
            step.num_requests, st.data_ptr(), st.stride(0), int(state_offset), self._stream()))

    # ---- norms in groups, depth mix, sums ---------------------------------------------------------
    def group_norm(self, x, weight, eps, groups, out=None, rows=None, residual=None):
        """RMS norm of every row of ``x`` in ``groups`` equal consecutive parts (each divided by its
        own ``sqrt(mean(part^2) + eps)``), times ``weight``: stored in ``out`` (of the rows ``rows``
        if given), or added to the float32 ``residual``."""
        n = x.shape[1]
        self._want(x.dtype == torch.float32 and x.is_contiguous() and weight.dtype == torch.float32
                   and weight.shape[0] == n, "group_norm: float32 rows and a float32 weight per element")
        self._want(n % groups == 0, f"group_norm: {n} elements do not fall into {groups} equal groups")
        num = x.shape[0] if rows is None else rows.shape[0]
        if residual is not None:
            self._want(rows is None and residual.dtype == torch.float32 and residual.stride(1) == 1
                       and tuple(residual.shape) == tuple(x.shape), "group_norm: a float32 residual of x's shape")
        else:
            self._want(out is not None and out.is_contiguous() and tuple(out.shape) == (num, n), "group_norm: out")
        self._rw(self.rows_lib.ti_group_norm_rows(
            x.data_ptr(), weight.data_ptr(), _ptr(rows), num, n, int(groups), float(eps), _ptr(out),
            _CODE[out.dtype] if out is not None else 0, _ptr(residual),
            residual.stride(0) if residual is not None else 0, self._stream()))

    def tanh_norm(self, x, alpha, weight, bias, out=None, rows=None, residual=None):
        """``tanh(alpha x) weight + bias`` for every row of the float32 ``x`` (one scalar ``alpha``, a
        weight and, if not None, a bias per element): stored in ``out`` (of the rows ``rows`` if given),
        or added to the float32 ``residual``."""
        n = x.shape[1]
        self._want(x.dtype == torch.float32 and x.is_contiguous() and weight.dtype == torch.float32
                   and weight.is_contiguous() and weight.shape[0] == n
                   and (bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.shape[0] == n)),
                   "tanh_norm: float32 rows, a float32 weight and bias per element")
        num = x.shape[0] if rows is None else rows.shape[0]
        if residual is not None:
            self._want(rows is None and residual.dtype == torch.float32 and residual.stride(1) == 1
                       and tuple(residual.shape) == tuple(x.shape), "tanh_norm: a float32 residual of x's shape")
        else:
            self._want(out is not None and out.is_contiguous() and tuple(out.shape) == (num, n)
                       and (rows is None or rows.dtype == torch.int32), "tanh_norm: out")
        self._rw(self.rows_lib.ti_tanh_norm_rows(
            x.data_ptr(), _ptr(rows), num, n, float(alpha), weight.data_ptr(), _ptr(bias), _ptr(out),
            _CODE[out.dtype] if out is not None else 0, _ptr(residual),
            residual.stride(0) if residual is not None else 0, self._stream()))

    def tanh_norm_pair(self, y, alpha1, weight1, bias1, residual, alpha2, weight2, bias2, out):
        """``residual += tanh(alpha1 y) weight1 + bias1``, then ``out = tanh(alpha2 residual) weight2 +
        bias2``: the norm behind one sublayer and the norm in front of the next, in one launch.  The
        float32 sum is the same as by ``tanh_norm`` twice."""
        n = y.shape[1]
        self._want(y.dtype == torch.float32 and y.is_contiguous() and residual.dtype == torch.float32
                   and residual.stride(1) == 1 and tuple(residual.shape) == tuple(y.shape) and out.is_contiguous()
                   and tuple(out.shape) == tuple(y.shape), "tanh_norm_pair: float32 rows, a residual and an output of their shape")
        for v in (weight1, bias1, weight2, bias2):
            self._want(v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.shape[0] == n),
                       "tanh_norm_pair: float32 weights and biases per element")
        self._rw(self.rows_lib.ti_tanh_norm_pair(
            y.data_ptr(), y.shape[0], n, float(alpha1), weight1.data_ptr(), _ptr(bias1), residual.data_ptr(),
            residual.stride(0), float(alpha2), weight2.data_ptr(), _ptr(bias2), out.data_ptr(), _CODE[out.dtype],
            self._stream()))

    def cap_rows(self, x, cap):
        """``x = cap tanh(x / cap)`` over a contiguous float32 tensor, in place."""
        self._want(x.dtype == torch.float32 and x.is_contiguous(), "cap_rows: contiguous float32")
        self._rw(self.rows_lib.ti_cap_rows(x.data_ptr(), x.numel(), float(cap), self._stream()))

    def add_row(self, x, row):
        """``x[t] += row`` for every row of the float32 ``x``."""
        self._want(x.dtype == torch.float32 and x.stride(1) == 1 and row.dtype == torch.float32 and row.is_contiguous()
                   and row.numel() == x.shape[1], "add_row: float32 rows and one float32 row of their length")
        self._rw(self.rows_lib.ti_add_row(x.data_ptr(), x.stride(0), row.data_ptr(), x.shape[0], x.shape[1],
                                           self._stream()))

    def depth_mix(self, x, hist, index, weights=None):
        """``hist[index] = x`` and, with ``weights`` (float32, ``index + 1`` of them),
        ``x = sum_{j <= index} weights[j] hist[j]``; ``x`` float32 ``[T, width]``, ``hist``
        ``[n, T, width]``."""
        self._want(x.dtype == torch.float32 and x.is_contiguous() and hist.dtype == torch.float32
                   and hist.is_contiguous() and tuple(hist.shape[1:]) == tuple(x.shape) and 0 <= index < hist.shape[0],
                   "depth_mix: float32 rows and a history of such rows")
        self._want(weights is None or (weights.dtype == torch.float32 and weights.is_contiguous()
                                       and weights.shape[0] == index + 1), "depth_mix: index + 1 float32 weights")
        self._rw(self.rows_lib.ti_depth_mix(x.data_ptr(), hist.data_ptr(), x.numel(), int(index), _ptr(weights),
                                             self._stream()))

    def add_scaled(self, dst, a, sa, b=None, sb=0.0):
        """``dst += sa * a [+ sb * b]`` over float32 rows."""
        self._want(dst.dtype == torch.float32 and dst.stride(1) == 1 and a.dtype == torch.float32 and a.is_contiguous()
                   and tuple(a.shape) == tuple(dst.shape)
                   and (b is None or (b.dtype == torch.float32 and b.is_contiguous() and b.shape == a.shape)),
                   "add_scaled: float32 rows of one shape")
        self._rw(self.rows_lib.ti_add_scaled(dst.data_ptr(), dst.stride(0), a.data_ptr(), float(sa), _ptr(b), float(sb),
                                              dst.shape[0], dst.shape[1], self._stream()))

    def glu_rows(self, gu, interleaved, kind, limit, alpha, out):
        """``out = act(gate, up)`` over the float32 product ``gu`` ``[T, 2 n]`` that holds gate and up
        columns stacked or, ``interleaved``, in strips of 8 and 8.  ``kind`` "silu": ``silu(g) u``;
        "clamped": ``g = min(g, limit)``, ``u = clamp(u, -limit, limit)``, ``g sigmoid(alpha g) (u + 1)``."""
        t, n = out.shape
        self._want(gu.dtype == torch.float32 and gu.is_contiguous() and tuple(gu.shape) == (t, 2 * n)
                   and out.is_contiguous(), "glu_rows: a float32 product of gate and up columns")
        self._rw(self.rows_lib.ti_glu_rows(gu.data_ptr(), t, n, int(bool(interleaved)), GLU_KINDS[kind], float(limit),
                                            float(alpha), out.data_ptr(), _CODE[out.dtype], self._stream()))

    # ---- recurrences over a matrix state -------------------------------------------------------------
    def matrix_state(self, mode, q, k, v, s0, s1, c0, c1, step, state, out, *, heads, kv_heads, dk, dv, eps,
                     norm_weight, norm_per_row=False, gate=None, gate_act="silu", cap=0.0):
        """One step of a recurrent mixer with a float32 matrix state ``[dk, dv]`` per head, for all
        tokens of the step in order, from and into each request's state slot (``state``: a
        ``StateView`` of ``matrix_state_floats`` floats).

        ``mode`` "delta" (the gated delta rule): ``q, k`` float32 rows of ``kv_heads x dk`` (brought to
        unit length here, q also times ``dk^-1/2``), ``v`` of ``heads x dv``; ``s0`` the logit of beta and
        ``s1`` the decay's argument per (token, head); ``c0 = A_log``, ``c1 = dt_bias`` per head.
        ``mode`` "gated_sum" (exponential gates under a running maximum): ``s0, s1`` the input and forget
        gates' pre-activations, ``c0, c1`` their biases, ``cap`` the bound of ``cap tanh(. / cap)``.

        Each head's output is brought to unit root mean square over ``dv`` (``eps``), multiplied by
        ``norm_weight`` (``[dv]``, or ``[heads * dv]`` with ``norm_per_row``) and by ``act(gate)``
        (float32 ``[T, heads * dv]``; "silu" or "sigmoid"), and written to ``out`` ``[T, heads * dv]``."""
        t = q.shape[0]
        st = state.state
        need = matrix_state_floats(mode, heads, dk, dv)
        for name, x, width in (("q", q, kv_heads * dk), ("k", k, kv_heads * dk), ("v", v, heads * dv),
                               ("s0", s0, heads), ("s1", s1, heads)):
            self._want(x.dtype == torch.float32 and x.stride(1) == 1 and x.shape[0] == t and x.shape[1] == width,
                       f"matrix_state: {name} must be float32 [T, {width}]")
        for name, x in (("c0", c0), ("c1", c1)):
            self._want(x.dtype == torch.float32 and x.is_contiguous() and x.shape[0] == heads,
                       f"matrix_state: {name} must hold one float32 per head")
        self._want(norm_weight.dtype == torch.float32 and norm_weight.is_contiguous()
                   and norm_weight.shape[0] == (heads * dv if norm_per_row else dv), "matrix_state: the norm's weight")
        self._want(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == t
                                    and gate.shape[1] == heads * dv), "matrix_state: the gate must be float32 [T, heads * dv]")
        self._want(st is not None and st.dtype == torch.float32 and st[0].numel() >= need and st.stride(-1) == 1,
                   f"matrix_state: the state must hold {need} float32 values per request")
        self._want(out.is_contiguous() and tuple(out.shape) == (t, heads * dv), "matrix_state: out")
        self._want(state.writes, "matrix_state: a recurrence renews its state")
        # few (request, head) pairs with long portions: a head's columns over several blocks
        col_block, o_raw, carry = 0, None, None
        pairs = step.num_requests * heads
        if dv > 128 or (self.cut_state_columns and dv >= 16 and step.max_q_len > 64 and pairs <= 2 * self.num_sms):
            col_block = 8
            while col_block < 128 and pairs * -(-dv // col_block) > 4 * self.num_sms:
                col_block *= 2
            o_raw = torch.empty((t, heads * dv), dtype=torch.float32, device=q.device)
            self.launches += 1
            if mode == "gated_sum":
                carry = torch.empty((pairs, dk + 1), dtype=torch.float32, device=q.device)
                self.launches += 1
        self._st(self.state_lib.ti_matrix_state(
            STATE_MODES[mode], q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
            s0.data_ptr(), s0.stride(0), s1.data_ptr(), s1.stride(0), c0.data_ptr(), c1.data_ptr(), float(cap),
            _ptr(gate), gate.stride(0) if gate is not None else 0, GATE_ACTS[gate_act], norm_weight.data_ptr(),
            int(bool(norm_per_row)), float(eps), step.cu_q.data_ptr(), state.slots.data_ptr(), step.num_requests, t,
            st.data_ptr(), st.stride(0), heads, kv_heads, dk, dv, col_block, out.data_ptr(), _CODE[out.dtype],
            _ptr(o_raw), _ptr(carry), self._stream()))
