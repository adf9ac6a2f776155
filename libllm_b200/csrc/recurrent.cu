// Kernels of mixers that carry fixed-size state from token to token: a short causal convolution
// over time on each channel, and the generalized delta rule (a matrix of state per head that
// decays per key channel, forgets along the current unit key and learns the outer product of key
// and value), with the norm and gate that follow it.  No counterpart in the reference, whose one
// mixer is attention (src/libllm/llama.cc:178-225).
//
// Everything that enters the recurrence is 32-bit: the projections arrive as the 32-bit results of
// their products, decays, removal rates, unit keys and the state itself are float.  A sequence's
// result depends on nothing but its own tokens and state: one thread owns one column of one head's
// state (or a fixed share of its rows), sums run in a fixed order, and no sum crosses sequences.
#include "common.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_recurrent_last_error)

// ---------------------------------------------------------------- causal convolution over time
// out_t = h_t + sum_j w[c, j] * h_(t - taps + 1 + j), zeros before the sequence's start.  The last
// taps - 1 inputs of every sequence are its state, state[slot][i][c] for the position
// length - (taps - 1) + i.  Rows whose window lies inside the step are computed by CTAs that own a
// run of rows (blockIdx.y < n_chunks); the first taps - 1 rows of each sequence, which need the
// state, by a CTA of their sequence (blockIdx.y - n_chunks), whose threads read the old state of
// their channel into registers before they write the new one: no other thread reads it.
constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_THREADS = 128;

template <int N>
__device__ __forceinline__ float pick(const float (&a)[N], int idx) {
  float r = 0.f;
#pragma unroll
  for (int k = 0; k < N; ++k)
    if (k == idx) r = a[k];
  return r;
}

// vals[j] = h at position p - taps + 1 + j; the same order of operations wherever a row is computed
__device__ __forceinline__ float conv_row(const float (&w)[CONV_MAX_TAPS], const float (&vals)[CONV_MAX_TAPS], int taps) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j)
    if (j < taps) s = fmaf(w[j], vals[j], s);
  return pick(vals, taps - 1) + s;
}

template <typename T>
__global__ void __launch_bounds__(CONV_THREADS)
causal_conv_kernel(const T *__restrict__ h, long long ldh, T *__restrict__ out, long long ldo, const float *__restrict__ weight,
                   T *__restrict__ state, const int *__restrict__ tok_seq, const int *__restrict__ tok_pos,
                   const int *__restrict__ seq_start, const int *__restrict__ seq_past, const int *__restrict__ seq_slot,
                   int n_tokens, int width, int taps, int n_chunks, int chunk_rows) {
  grid_dependents_launch();
  const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
  float w[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) w[j] = (c < width && j < taps) ? weight[(size_t)c * taps + j] : 0.f;
  grid_dependency_wait();
  if (c >= width) return;
  const int keep = taps - 1;
  float vals[CONV_MAX_TAPS];
  if ((int)blockIdx.y < n_chunks) {
    const int r0 = blockIdx.y * chunk_rows, r1 = min(n_tokens, r0 + chunk_rows);
    for (int row = r0; row < r1; ++row) {
      const int b = tok_seq[row];
      if (tok_pos[row] - seq_past[b] < keep) continue;          // the sequence's own CTA computes it
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j)
        vals[j] = j < taps ? to_float(h[(size_t)(row - keep + j) * ldh + c]) : 0.f;
      out[(size_t)row * ldo + c] = from_float<T>(conv_row(w, vals, taps));
    }
    return;
  }
  const int b = blockIdx.y - n_chunks;
  const int start = seq_start[b], n = seq_start[b + 1] - start;
  T *st = state + (size_t)seq_slot[b] * keep * width + c;
  float old[CONV_MAX_TAPS - 1];
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) old[i] = i < keep ? to_float(st[(size_t)i * width]) : 0.f;
  // position (relative to the sequence's length before the step) -> input
  auto at = [&](int rel) { return rel < 0 ? pick(old, keep + rel) : to_float(h[(size_t)(start + rel) * ldh + c]); };
  for (int i = 0; i < min(n, keep); ++i) {
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) vals[j] = j < taps ? at(i - keep + j) : 0.f;
    out[(size_t)(start + i) * ldo + c] = from_float<T>(conv_row(w, vals, taps));
  }
  for (int i = 0; i < keep; ++i) st[(size_t)i * width] = from_float<T>(at(n - keep + i));
}

LLM_EXPORT int llm_causal_conv(int dtype, const void *h, long long ldh, void *out, long long ldo, const float *weight, void *state,
                               const int *tok_seq, const int *tok_pos, const int *seq_start, const int *seq_past,
                               const int *seq_slot, int n_tokens, int n_seqs, int width, int taps, int single_tokens,
                               cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_seqs > 0 && width > 0, "causal_conv: bad sizes");
  LLM_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "causal_conv: %d taps are not supported (1 to %d)", taps, CONV_MAX_TAPS);
  LLM_REQUIRE(taps == 1 || state != nullptr, "causal_conv: a convolution of %d taps needs its state", taps);
  const int chunk_rows = 8;
  // a step of single tokens has no row whose window lies inside the step (but for one tap)
  const int n_chunks = single_tokens && taps > 1 ? 0 : (n_tokens + chunk_rows - 1) / chunk_rows;
  const int n_own = taps > 1 ? n_seqs : 0;
  if (n_chunks + n_own == 0) return LLM_OK;
  LLM_REQUIRE(n_chunks + n_own <= 65535, "causal_conv: too many rows for one launch");
  const dim3 grid((width + CONV_THREADS - 1) / CONV_THREADS, n_chunks + n_own);
  if (dtype == LLM_F32)
    llm_launch(causal_conv_kernel<float>, grid, dim3(CONV_THREADS), 0, stream, (const float *)h, ldh, (float *)out, ldo, weight,
               (float *)state, tok_seq, tok_pos, seq_start, seq_past, seq_slot, n_tokens, width, taps, n_chunks, chunk_rows);
  else if (dtype == LLM_BF16)
    llm_launch(causal_conv_kernel<__nv_bfloat16>, grid, dim3(CONV_THREADS), 0, stream, (const __nv_bfloat16 *)h, ldh,
               (__nv_bfloat16 *)out, ldo, weight, (__nv_bfloat16 *)state, tok_seq, tok_pos, seq_start, seq_past, seq_slot, n_tokens,
               width, taps, n_chunks, chunk_rows);
  else LLM_FAIL("causal_conv: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("causal_conv");
  return LLM_OK;
}

// ---------------------------------------------------------------- the delta rule: what each token brings
// From a token's projections (32-bit rows of the stacked product: r, k, v, ..., the removal
// logits and the low-rank decay input) to the vectors of the recurrence, per head and key channel:
//   decay   w = exp(-decay_scale * sigmoid(w0 + W2 tanh(x1)))       x1 = the low-rank projection
//   unit    u = k / sqrt(sum(k^2) + key_eps)
//   removal b = sigmoid(a + a_bias) * u
// prep [tokens, heads, 3, d]: w, b, u.  One warp per (token, head); sums over the head in lane
// order then the shuffle tree, whatever the launch.
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float *__restrict__ proj, long long ld, int off_k, int off_a, int off_x1, int rank,
                     const float *__restrict__ w2, const float *__restrict__ w0, const float *__restrict__ a_bias,
                     float decay_scale, float key_eps, int n_tokens, int n_heads, int d, float *__restrict__ prep) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * n_heads) return;
  const int t = (int)(item / n_heads), hd = (int)(item - (long long)t * n_heads);
  const float *row = proj + (size_t)t * ld;
  const float *k = row + off_k + (size_t)hd * d;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) ss = fmaf(k[i], k[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss + key_eps);
  float *o = prep + (size_t)item * 3 * d;
  for (int i = lane; i < d; i += 32) {
    const int ch = hd * d + i;
    float z = w0[ch];
    const float *w2r = w2 + (size_t)ch * rank;
    for (int q = 0; q < rank; ++q) z = fmaf(w2r[q], tanhf(row[off_x1 + q]), z);
    const float u = k[i] * inv;
    const float a = 1.f / (1.f + expf(-(row[off_a + ch] + a_bias[ch])));
    o[i] = expf(-decay_scale / (1.f + expf(-z)));
    o[d + i] = a * u;
    o[2 * d + i] = u;
  }
}

// ---------------------------------------------------------------- the delta rule: the recurrence
// Per head, state S [d keys x d values]:  S <- diag(w) S - b (u^T S) + k v^T  (both terms read the
// old S), then o = S^T r.  A column of S never meets another column, so a thread (or LANES
// neighbouring lanes, each with d / LANES of the rows) owns column j for the whole step and walks
// the sequence's tokens in order; the token's vectors are staged in shared memory, the next token's
// loads issued before this token's arithmetic.  state[slot][head][j][i] (a column's rows together).
constexpr int DR_THREADS = 64;

template <int DMAX, int LANES>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float *__restrict__ proj, long long ld, int off_r, int off_k, int off_v,
                  const float *__restrict__ prep, float *__restrict__ state, float *__restrict__ out, long long ldo,
                  const int *__restrict__ seq_start, const int *__restrict__ seq_slot, int n_heads, int d) {
  constexpr int ROWS = DMAX / LANES;                 // rows of a column held by one thread
  constexpr int COLS = DR_THREADS / LANES;           // columns of a CTA
  __shared__ __align__(16) float vec[2][5][DMAX];    // w, b, u, k, r of a token, two tokens in turn
  __shared__ float vcol[2][COLS];
  grid_dependents_launch();
  grid_dependency_wait();
  const int b = blockIdx.x, hd = blockIdx.y;
  const int tid = threadIdx.x, sub = tid % LANES, col = tid / LANES;
  const int j = blockIdx.z * COLS + col;
  const int start = seq_start[b], n = seq_start[b + 1] - start;
  const bool live = j < d;
  float S[ROWS];
  float *sp = state + (((size_t)seq_slot[b] * n_heads + hd) * d + (live ? j : 0)) * d + sub * ROWS;
#pragma unroll
  for (int i = 0; i < ROWS; ++i) S[i] = (live && sub * ROWS + i < d) ? sp[i] : 0.f;

  // what this thread stages for a token: elements tid, tid + DR_THREADS, ... of the five vectors
  constexpr int PER = (5 * DMAX + DR_THREADS - 1) / DR_THREADS;
  float stage[PER], stage_v = 0.f;
  auto fetch = [&](int t) {
    const float *row = proj + (size_t)(start + t) * ld;
    const float *pr = prep + ((size_t)(start + t) * n_heads + hd) * 3 * d;
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int idx = tid + e * DR_THREADS, which = idx / DMAX, i = idx - which * DMAX;
      float v = 0.f;
      if (which < 5 && i < d) v = which < 3 ? pr[which * d + i] : row[(which == 3 ? off_k : off_r) + hd * d + i];
      stage[e] = v;
    }
    if (tid < COLS) stage_v = blockIdx.z * COLS + tid < d ? row[off_v + hd * d + blockIdx.z * COLS + tid] : 0.f;
  };
  auto put = [&](int buf) {
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int idx = tid + e * DR_THREADS, which = idx / DMAX, i = idx - which * DMAX;
      if (which < 5) vec[buf][which][i] = stage[e];
    }
    if (tid < COLS) vcol[buf][tid] = stage_v;
  };
  if (n > 0) {
    fetch(0);
    put(0);
  }
  __syncthreads();
  for (int t = 0; t < n; ++t) {
    const int buf = t & 1;
    if (t + 1 < n) fetch(t + 1);
    const float *w = vec[buf][0] + sub * ROWS, *bb = vec[buf][1] + sub * ROWS, *u = vec[buf][2] + sub * ROWS;
    const float *k = vec[buf][3] + sub * ROWS, *r = vec[buf][4] + sub * ROWS;
    const float v = vcol[buf][col];
    float us = 0.f;
#pragma unroll
    for (int i = 0; i < ROWS; ++i) us = fmaf(u[i], S[i], us);
#pragma unroll
    for (int o = 1; o < LANES; o <<= 1) us += __shfl_xor_sync(0xffffffffu, us, o);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      S[i] = fmaf(w[i], S[i], fmaf(k[i], v, -bb[i] * us));
      acc = fmaf(S[i], r[i], acc);
    }
#pragma unroll
    for (int o = 1; o < LANES; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (live && sub == 0) out[(size_t)(start + t) * ldo + (size_t)hd * d + j] = acc;
    if (t + 1 < n) put(buf ^ 1);
    __syncthreads();
  }
  if (live)
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
      if (sub * ROWS + i < d) sp[i] = S[i];
}

LLM_EXPORT int llm_delta_rule(const float *proj, long long ld, int off_r, int off_k, int off_v, int off_a, int off_x1, int rank,
                              const float *w2, const float *w0, const float *a_bias, float decay_scale, float key_eps,
                              float *prep, float *state, float *out, long long ldo, const int *seq_start, const int *seq_slot,
                              int n_tokens, int n_seqs, int n_heads, int d, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_seqs > 0 && n_heads > 0 && d > 0 && rank > 0, "delta_rule: bad sizes");
  LLM_REQUIRE(d <= 256, "delta_rule: heads of %d channels are not supported (up to 256)", d);
  LLM_REQUIRE(n_heads <= 65535 && n_seqs < 2147483647, "delta_rule: too many heads or sequences");
  const long long items = (long long)n_tokens * n_heads;
  llm_launch(delta_prepare_kernel, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, proj, ld, off_k, off_a, off_x1, rank, w2,
             w0, a_bias, decay_scale, key_eps, n_tokens, n_heads, d, prep);
  LLM_CHECK_LAUNCH("delta_prepare");
#define DR_GO(DMAX, LANES)                                                                                              \
  llm_launch(delta_rule_kernel<DMAX, LANES>, dim3(n_seqs, n_heads, (d + DR_THREADS / LANES - 1) / (DR_THREADS / LANES)), \
             dim3(DR_THREADS), 0, stream, proj, ld, off_r, off_k, off_v, (const float *)prep, state, out, ldo, seq_start, \
             seq_slot, n_heads, d)
  if (d <= 32) DR_GO(32, 2);
  else if (d <= 64) DR_GO(64, 4);
  else if (d <= 128) DR_GO(128, 4);
  else DR_GO(256, 8);
#undef DR_GO
  LLM_CHECK_LAUNCH("delta_rule");
  return LLM_OK;
}

// ---------------------------------------------------------------- norm per head, weight, gate
// out[t, h, :] = x[t, h, :] / sqrt(mean(x[t, h, :]^2) + eps) * weight[h, :] * sigmoid(gate[t, h, :])
// eps < 0: no norm; weight null: none; gate null: none (gate: 32-bit logits, row stride gate_stride).
// One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float *__restrict__ x, long long ldx, const float *__restrict__ weight, const float *__restrict__ gate,
                      long long gate_stride, float eps, int n_tokens, int n_heads, int dv, T *__restrict__ out, long long ldo) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * n_heads) return;
  const int t = (int)(item / n_heads), hd = (int)(item - (long long)t * n_heads);
  const float *xr = x + (size_t)t * ldx + (size_t)hd * dv;
  float inv = 1.f;
  if (eps >= 0.f) {
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(xr[i], xr[i], ss);
    ss = warp_sum(ss);
    inv = 1.f / sqrtf(ss / (float)dv + eps);
  }
  for (int i = lane; i < dv; i += 32) {
    float v = xr[i] * inv;
    if (weight) v *= weight[(size_t)hd * dv + i];
    if (gate) v *= 1.f / (1.f + expf(-gate[(size_t)t * gate_stride + (size_t)hd * dv + i]));
    out[(size_t)t * ldo + (size_t)hd * dv + i] = from_float<T>(v);
  }
}

LLM_EXPORT int llm_head_norm_gate(const float *x, long long ldx, const float *weight, const float *gate, long long gate_stride,
                                  float eps, int n_tokens, int n_heads, int dv, void *out, int out_dtype, long long ldo,
                                  cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && dv > 0 && x && out, "head_norm_gate: bad arguments");
  const long long items = (long long)n_tokens * n_heads;
  const dim3 grid((unsigned)((items + 3) / 4));
  if (out_dtype == LLM_F32)
    llm_launch(head_norm_gate_kernel<float>, grid, dim3(128), 0, stream, x, ldx, weight, gate, gate_stride, eps, n_tokens, n_heads, dv,
               (float *)out, ldo);
  else if (out_dtype == LLM_BF16)
    llm_launch(head_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, x, ldx, weight, gate, gate_stride, eps, n_tokens,
               n_heads, dv, (__nv_bfloat16 *)out, ldo);
  else LLM_FAIL("head_norm_gate: unknown dtype %d", out_dtype);
  LLM_CHECK_LAUNCH("head_norm_gate");
  return LLM_OK;
}
