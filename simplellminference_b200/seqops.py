"""Python face of the ragged-token-batch launchers (sllm_seq_* of include/sllm_b200.h), in the manner of kernels.py: torch tensors only
carry device memory, every function enqueues one kernel (or a short fixed sequence) on the stream it is given and returns. There is no
fallback: the launchers raise if the CUDA library is missing or a call fails.

Additive to the reference (one Llama forward, source/model/model.cpp:40-140): these are the blocks of models that mix softmax attention
over a paged cache with recurrent layers."""
from __future__ import annotations

import ctypes as C

from . import _lib
from .config import BF16, F32

_NULL = None


def _p(t):
    return None if t is None else t.data_ptr()


class Ops:
    """Bound launchers + the numeric mode of a run: ``w_dtype`` is the storage type of the matrices, ``round_a`` rounds activations to bf16
    as matrix-product operands (the bf16 mode), ``kv_dtype`` the type of the attention pools."""

    def __init__(self, w_dtype: int, build: bool = False):
        self.lib = _lib.load_seq(build=build)
        self.w_dtype = w_dtype
        self.round_a = 1 if w_dtype == BF16 else 0
        self.kv_dtype = BF16 if w_dtype == BF16 else F32
        self.tensor_cores = w_dtype == BF16
        self.launches = 0

    def _ck(self, rc):
        self.launches += 1
        if rc != 0:
            raise _lib.SllmError(rc, self.lib.sllm_last_error().decode(errors="replace"))

    # ---- rows ----
    def embed(self, ids, table, vocab, d, streams, out, T, st, scale=1.0):
        self._ck(self.lib.sllm_seq_embed(_p(ids), _p(table), self.w_dtype, vocab, d, streams, scale, _p(out), T, st))

    def layernorm(self, x, ldx, w, bias, eps, y, ldy, T, d, st, y16=None):
        self._ck(self.lib.sllm_seq_layernorm(_p(x), ldx, _p(w), _p(bias), eps, _p(y), ldy, _p(y16), T, d, st))

    def depth_average(self, x, y, hist, n_prev, coef, norm_w, norm_b, eps, h, T, d, st, h16=None):
        self._ck(self.lib.sllm_seq_depth_average(_p(x), _p(y), _p(hist), n_prev, _p(coef), _p(norm_w), _p(norm_b), eps, _p(h), _p(h16), T, d, st))

    def clamped_glu(self, gate_ptr, ldg, up_ptr, ldu, limit, alpha, out, ldo, T, n, st, out16=None):
        self._ck(self.lib.sllm_seq_clamped_glu(gate_ptr, ldg, up_ptr, ldu, limit, alpha, _p(out), ldo, _p(out16), T, n, st))

    def on_tensor_cores(self, T, N, K, ldw=None, batch=1):
        """Whether ``linear`` with a bf16 scratch sends this product to the tensor cores (then a producer may leave the operand there)."""
        return bool(self.tensor_cores and self.lib.sllm_seq_linear_on_tensor_cores(T, N, K, self.w_dtype, K if ldw is None else ldw, batch, self.round_a))

    def hyper_read(self, x, streams, T, d, coef, norm_w, groups, eps, y, st):
        self._ck(self.lib.sllm_seq_hyper_read(_p(x), streams, T, d, _p(coef), _p(norm_w), groups, eps, _p(y), st))

    def hyper_write(self, x, streams, T, d, mix, outc, y, st):
        self._ck(self.lib.sllm_seq_hyper_write(_p(x), streams, T, d, _p(mix), _p(outc), _p(y), st))

    def hyper_write_read(self, x, streams, T, d, mix, outc, y_in, coef, norm_w, groups, eps, y_out, st):
        self._ck(self.lib.sllm_seq_hyper_write_read(_p(x), streams, T, d, _p(mix), _p(outc), _p(y_in), _p(coef), _p(norm_w), groups, eps, _p(y_out), st))

    def linear(self, a_ptr, lda, w, ldw, bias, c_ptr, ldc, T, N, K, st, alpha=1.0, accumulate=False, batch=1, a_bs=0, w_bs=0, bias_bs=0,
               c_bs=0, scratch=None, a16_ready=False, rows_dev=None, w_ptr=None):
        """``w_ptr``: an address inside ``w`` to use instead of its start (one matrix of several stored back to back);
        ``rows_dev``: device address of a row count, rows beyond it are skipped."""
        self._ck(self.lib.sllm_seq_linear(a_ptr, lda, _p(w) if w_ptr is None else w_ptr, self.w_dtype, ldw, _p(bias), c_ptr, ldc, T, N, K, alpha, int(accumulate),
                                          self.round_a, batch, a_bs, w_bs, bias_bs, c_bs,
                                          (scratch if isinstance(scratch, int) else _p(scratch)) if self.tensor_cores else None, int(a16_ready), rows_dev, st))

    def polynorm(self, z, ldz, coef, eps, out, ldo, T, n, st):
        self._ck(self.lib.sllm_seq_polynorm(_p(z), ldz, _p(coef), eps, _p(out), ldo, T, n, st))

    def gather_rows(self, x, ldx, rows, n, d, out, st):
        self._ck(self.lib.sllm_seq_gather_rows(_p(x), ldx, _p(rows), n, d, _p(out), st))

    def headnorm_gate(self, o_ptr, ldo, g_ptr, ldg, w, heads, dv, eps, out, ldout, T, st, out16=None, gate_first=False, wide_weight=False):
        """``gate_first``: the gate multiplies before the norm; ``wide_weight``: w holds heads * dv entries instead of dv."""
        self._ck(self.lib.sllm_seq_headnorm_gate(o_ptr, ldo, g_ptr, ldg, _p(w), heads, dv, eps, _p(out), ldout, _p(out16), T,
                                                 int(bool(gate_first)) | 2 * int(bool(wide_weight)), st))

    # ---- attention over the paged cache ----
    def rotary_kv(self, b, q_ptr, ldq, heads, dk, k_ptr, ldk, kv_heads, v_ptr, ldv, dv, freq, n_freq, magnitude, vfreq, layout, k_pool, v_pool, st):
        self._ck(self.lib.sllm_seq_rotary_kv(C.byref(b), q_ptr, ldq, heads, dk, k_ptr, ldk, kv_heads, v_ptr, ldv, dv, _p(freq), n_freq, magnitude,
                                             _p(vfreq), layout, _p(k_pool), _p(v_pool), self.kv_dtype, st))

    def attention(self, b, q_ptr, ldq, heads, kv_heads, dk, dv, scale, k_pool, v_pool, nsplit, ws, st, opts=None):
        self._ck(self.lib.sllm_seq_attention(C.byref(b), q_ptr, ldq, heads, kv_heads, dk, dv, scale, _p(k_pool), _p(v_pool), self.kv_dtype, nsplit,
                                             _p(ws), C.byref(opts) if opts is not None else None, st))

    def attention_finish(self, b, ws, nsplit, heads, dv, vfreq, layout, gate_ptr, ldg, out, ldo, st, sink=None):
        self._ck(self.lib.sllm_seq_attention_finish(C.byref(b), _p(ws), nsplit, heads, dv, _p(vfreq), layout, gate_ptr, ldg, _p(sink), _p(out), ldo, st))

    @staticmethod
    def attention_options(window=0, keep_first=0, softcap=0.0, slopes=None, values_in_keys=False, logdist=None, cross_values=False):
        """The options structure of ``attention``; the caller keeps the ``slopes`` and ``logdist`` tensors alive."""
        return _lib.SeqAttnOpts(int(window or 0), int(keep_first or 0), float(softcap or 0.0), _p(slopes), int(bool(values_in_keys)), _p(logdist),
                                int(bool(cross_values)))

    def normed_rotary_kv(self, b, q_ptr, ldq, heads, dk, k_ptr, ldk, kv_heads, v_ptr, ldv, dv, q_norm_w, k_norm_w, eps, freq, n_freq, layout, k_pool, v_pool, st):
        self._ck(self.lib.sllm_seq_normed_rotary_kv(C.byref(b), q_ptr, ldq, heads, dk, k_ptr, ldk, kv_heads, v_ptr, ldv, dv, _p(q_norm_w), _p(k_norm_w), eps,
                                                    _p(freq), n_freq, layout, _p(k_pool), _p(v_pool), self.kv_dtype, st))

    def head_mix(self, x, ldx, mix, heads, kv_heads, dv, out, ldo, T, st, out16=None):
        self._ck(self.lib.sllm_seq_head_mix(_p(x), ldx, _p(mix), heads, kv_heads, dv, _p(out), ldo, _p(out16), T, st))

    def unit_kv(self, b, q_ptr, ldq, heads, dk, k_ptr, ldk, kv_heads, v_ptr, ldv, dv, eps, unit, v_shared, share, lam, k_pool, v_pool, st,
                q_temp_coef=0.0, q_temp_every=0):
        self._ck(self.lib.sllm_seq_unit_kv(C.byref(b), q_ptr, ldq, heads, dk, k_ptr, ldk, kv_heads, v_ptr, ldv, dv, eps, unit, _p(v_shared), share, lam,
                                           _p(k_pool), _p(v_pool), self.kv_dtype, q_temp_coef, q_temp_every, st))

    def latent_kv(self, b, q_ptr, ldq, heads, dn, dr, low_ptr, ldlow, rank, norm_w, eps, freq, n_freq, q_out, ldqo, pool, st, magnitude=1.0):
        """``low_ptr`` None: nothing is cached (the pool belongs to another layer), only the queries' rotated parts are produced."""
        self._ck(self.lib.sllm_seq_latent_kv(C.byref(b), q_ptr, ldq, heads, dn, dr, low_ptr, ldlow, rank, _p(norm_w), eps, _p(freq), n_freq, _p(q_out),
                                             ldqo, _p(pool) if low_ptr else None, self.kv_dtype, magnitude, st))

    # ---- scalar norms around sublayers that read through a short convolution ----
    def embed_pair(self, ids, prev_ids, table, pairs, vocab, d, buckets, mul_prev, mul_cur, out, T, st):
        self._ck(self.lib.sllm_seq_embed_pair(_p(ids), _p(prev_ids), _p(table), _p(pairs), self.w_dtype, vocab, d, buckets, mul_prev, mul_cur, _p(out), T, st))

    def seam(self, b, x_in, d, st, x_out=None, y=None, post_g=1.0, pre_g=None, eps=0.0, conv_w=None, taps=1, ring=None, h=None, h16=None, stash=None,
             flush_ring=None, flush_taps=0, scales=None, post_norm=True, pre_w=None, pre_w_offset=0.0):
        """x_out = x_in + post_g * y / rms(y) (if ``y``; ``post_norm`` False: x_in + y), then h = n + conv(n), n = pre_g * x / rms(x) (if
        ``pre_g`` is given), times (pre_w_offset + pre_w) per channel if ``pre_w`` is."""
        self._ck(self.lib.sllm_seq_seam(C.byref(b), _p(x_in), _p(x_out), _p(y), post_g, int(pre_g is not None), pre_g or 0.0, eps, _p(conv_w), taps, _p(ring),
                                        _p(h), _p(h16), _p(stash), _p(flush_ring), flush_taps, d, _p(scales), int(bool(post_norm)), _p(pre_w), pre_w_offset, st))

    def rmsnorm_rows(self, x_ptr, ldx, w, eps, y_ptr, ldy, T, n, st):
        self._ck(self.lib.sllm_seq_rmsnorm_rows(x_ptr, ldx, _p(w), eps, y_ptr, ldy, T, n, st))

    def gated_act(self, gate_ptr, ldg, up_ptr, ldu, out, ldo, T, n, st, out16=None, act=0):
        self._ck(self.lib.sllm_seq_gated_act(gate_ptr, ldg, up_ptr, ldu, act, _p(out), ldo, _p(out16), T, n, st))

    def softcap(self, x, n, cap, st):
        self._ck(self.lib.sllm_seq_softcap(_p(x), n, cap, st))

    def moe_act(self, logits_ptr, ldl, n_route, experts, top, correction, up_ptr, ldu, ff, act, h, ldh, d, out, out16, y, ldy, T, st, route_w=None):
        self._ck(self.lib.sllm_seq_moe_act(logits_ptr, ldl, n_route, experts, top, _p(correction), up_ptr, ldu, ff, act, _p(h), ldh, d, _p(out), _p(out16),
                                           _p(y), ldy, _p(route_w), T, st))

    # ---- mixture of experts with the tokens gathered per expert ----
    def zero(self, ptr, n_bytes, st):
        self._ck(self.lib.sllm_seq_zero(ptr, n_bytes, st))

    def moe_route(self, logits_ptr, ldl, n_route, experts, top, correction, h, ldh, d, counts_ptr, cap, sel_e, sel_pos, sel_w, ident, rows16, rows32, T, st,
                  mode=0):
        self._ck(self.lib.sllm_seq_moe_route(logits_ptr, ldl, n_route, experts, top, _p(correction), _p(h), ldh, d, counts_ptr, cap, sel_e, sel_pos, sel_w, ident,
                                             rows16, rows32, T, mode, st))

    def act(self, x_ptr, n, kind, st):
        self._ck(self.lib.sllm_seq_act(x_ptr, n, kind, st))

    def linear_indexed(self, a_ptr, lda, a_bs, a_div, w, ldw, w_bs, w_index, c_ptr, ldc, c_bs, batch, N, K, st):
        """``batch`` products of one row each, product b with the matrix ``w_index[b]`` (device array) of ``w``."""
        self._ck(self.lib.sllm_seq_linear_indexed(a_ptr, lda, a_bs, a_div, _p(w), self.w_dtype, ldw, w_bs, w_index, c_ptr, ldc, c_bs, batch, N, K, self.round_a, st))

    def moe_expert_act(self, up_ptr, counts_ptr, experts, cap, ff, act, out16, out32, st):
        self._ck(self.lib.sllm_seq_moe_expert_act(up_ptr, counts_ptr, experts, cap, ff, act, out16, out32, st))

    def moe_pair_act(self, up_ptr, sel_w_ptr, pairs, ff, act, out_ptr, w_out_ptr, st):
        self._ck(self.lib.sllm_seq_moe_pair_act(up_ptr, sel_w_ptr, pairs, ff, act, out_ptr, w_out_ptr, st))

    def moe_combine(self, down_ptr, sel_e, sel_pos, sel_w, top, ident, h, ldh, cap, d, y, ldy, T, st):
        self._ck(self.lib.sllm_seq_moe_combine(down_ptr, sel_e, sel_pos, sel_w, top, ident, _p(h), ldh, cap, d, _p(y), ldy, T, st))

    # ---- recurrences ----
    def conv_ring(self, b, x_ptr, ldx, channels, taps, w, ring, act, out, ldo, st, bias=None):
        self._ck(self.lib.sllm_seq_conv_ring(C.byref(b), x_ptr, ldx, channels, taps, _p(w), _p(bias), _p(ring), act, _p(out), ldo, st))

    def ring_store(self, b, x_ptr, ldx, channels, taps, ring, st):
        self._ck(self.lib.sllm_seq_ring_store(C.byref(b), x_ptr, ldx, channels, taps, _p(ring), st))

    def ssd_scan(self, b, x_ptr, ldx, B_ptr, ldb, C_ptr, ldc, step_ptr, lda, a_log, dt_bias, skip, heads, groups, n_state, dv, state, y, ldy, conv_x_ptr, ld_conv,
                 channels, taps, ring, st, scratch=None):
        self._ck(self.lib.sllm_seq_ssd_scan(C.byref(b), x_ptr, ldx, B_ptr, ldb, C_ptr, ldc, step_ptr, lda, _p(a_log), _p(dt_bias), _p(skip), heads, groups, n_state,
                                            dv, _p(state), _p(y), ldy, conv_x_ptr, ld_conv, channels, taps, _p(ring), _p(scratch), st))

    def selective_scan(self, b, x_ptr, ldx, step_ptr, lddt, B_ptr, ldb, C_ptr, ldc, z_ptr, ldz, a_log, skip, inner, n_state, state, out, ldo, conv_x_ptr, ld_conv,
                       taps, ring, st, out16=None, scratch=None):
        self._ck(self.lib.sllm_seq_selective_scan(C.byref(b), x_ptr, ldx, step_ptr, lddt, B_ptr, ldb, C_ptr, ldc, z_ptr, ldz, _p(a_log), _p(skip), inner, n_state,
                                                  _p(state), _p(out), ldo, _p(out16), conv_x_ptr, ld_conv, taps, _p(ring), _p(scratch), st))

    def delta_rule(self, b, q_ptr, ldq, k_ptr, ldk, v_ptr, ldv, beta_ptr, ldb, step_ptr, lda, a_log, dt_bias, heads, kv_heads, dk, dv, unit_eps, qscale,
                   state, o, ldo, conv_x_ptr, ldx, channels, taps, ring, st):
        self._ck(self.lib.sllm_seq_delta_rule(C.byref(b), q_ptr, ldq, k_ptr, ldk, v_ptr, ldv, beta_ptr, ldb, step_ptr, lda, _p(a_log), _p(dt_bias), heads,
                                              kv_heads, dk, dv, unit_eps, qscale, _p(state), _p(o), ldo, conv_x_ptr, ldx, channels, taps, _p(ring), st))

    def conv(self, b, x_ptr, ldx, channels, taps, w, cb, tail, u, ldu, st):
        self._ck(self.lib.sllm_seq_conv(C.byref(b), x_ptr, ldx, channels, taps, _p(w), _p(cb), _p(tail), _p(u), ldu, st))

    def rglru_scan(self, b, u, ldu, lr_ptr, li_ptr, ldg, y_ptr, ldy, lam, c, channels, state, x_ptr, ldx, taps, tail, out, ldo, scratch, st):
        self._ck(self.lib.sllm_seq_rglru_scan(C.byref(b), _p(u), ldu, lr_ptr, li_ptr, ldg, y_ptr, ldy, _p(lam), c, channels, _p(state), x_ptr, ldx,
                                              taps, _p(tail), _p(out), ldo, _p(scratch), st))

    def gla_scan(self, b, q_ptr, ldq, k_ptr, ldk, v_ptr, ldv, z_ptr, ldz, heads, dk, dv, qscale, tau, state, o, ldo, scratch, st):
        self._ck(self.lib.sllm_seq_gla_scan(C.byref(b), q_ptr, ldq, k_ptr, ldk, v_ptr, ldv, z_ptr, ldz, heads, dk, dv, qscale, tau, _p(state),
                                            _p(o), ldo, _p(scratch), st))

    # ---- sampling (the op of the one-sequence path: temperature <= 0 = first maximum) ----
    def sample(self, logits_ptr, n, temperature, top_k, top_p, seed, step, idx_ptr, st):
        self._ck(self.lib.sllm_sample_f32(logits_ptr, n, temperature, top_k, top_p, seed, step, idx_ptr, st))
