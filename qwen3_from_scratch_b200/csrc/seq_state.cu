// Mixers that carry a state of fixed size from token to token instead of a cache of keys: the pieces they
// are made of.  Every piece works on a mixed batch (rows of the batch are requests, each with a portion of
// one or more tokens, `q_start[b] .. q_start[b + 1]`), reads what earlier steps left in the request's state
// slot (`slot_ids[b]`) and leaves there what later steps need, so that a prompt cut anywhere gives the same
// numbers as the whole prompt: all recurrences are evaluated token by token in float32, in the same order
// whatever the cut.
//
//   token_shift       h_t = x_t + (x_{t-1} - x_t) * mu       (x_{-1} = 0; the state is the last x)
//   causal_conv       u_t = act(sum_j w[c, j] * v_{t-(K-1-j)} + b),  v = x + in_bias (zeros before the start;
//                     the state is the last K - 1 inputs v), one channel per filter
//   block_diag_gates  per block of channels: G_t = W_b u_t,b  (two square matrices per block, stacked)
//   rglru_scan        a_t = exp(-c * softplus(lam) * r_t),  S_t = a_t S_{t-1} + sqrt(1 - a_t^2) i_t u_t,
//                     r, i = sigmoid(G + bias);  out = S_t * gelu_tanh(y_t + bias)
//   selective_scan    S_t[c, n] = exp(dt_t,c A[c, n]) S_{t-1}[c, n] + dt_t,c x_t,c B_t,n,
//                     y_t,c = sum_n S_t[c, n] C_t,n + D_c x_t,c;  out = y * silu(z)
//
// A slot id outside the pool sets the BAD_POSITION bit and the row is left out; nothing faults.
#include "common.cuh"

namespace q3 {

// ---------------------------------------------------------------- token shift
// One block per token.  The block of a request's first token of the step reads the state (the x of the
// token before) and, element by element after reading it, stores the portion's last x there.
template <typename T>
__global__ void token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mu, float* __restrict__ state,
                                   const int* __restrict__ q_start, const int* __restrict__ tok_seq,
                                   const int* __restrict__ slot_ids, T* __restrict__ out, int W, int num_slots,
                                   int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  const int slot = slot_ids[b];
  const float* cur = x + (size_t)t * W;
  T* o = out + (size_t)t * W;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    for (int i = threadIdx.x; i < W; i += blockDim.x) o[i] = from_float<T>(0.f);
    return;
  }
  if (t == q_start[b]) {
    float* st = state + (size_t)slot * W;
    const float* last = x + (size_t)(q_start[b + 1] - 1) * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float c = cur[i], p = st[i];
      o[i] = from_float<T>(c + (p - c) * mu[i]);
      st[i] = last[i];
    }
  } else {
    const float* prev = cur - W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float c = cur[i];
      o[i] = from_float<T>(c + (prev[i] - c) * mu[i]);
    }
  }
}

// ---------------------------------------------------------------- short causal convolution per channel
// grid (tokens, channel chunks).  x: [T, ldx] with the C channels at column x_col; state: [slots, K - 1, C]
// float32, entry K - 2 the newest.  The state is only read here; conv_state_kernel renews it afterwards.
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ in_bias,
                                   const float* __restrict__ w, const float* __restrict__ bias,
                                   const float* __restrict__ state, const int* __restrict__ q_start,
                                   const int* __restrict__ tok_seq, const int* __restrict__ slot_ids,
                                   T* __restrict__ out, int C, int K, int act, int num_slots, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = tok_seq[t];
  const int slot = slot_ids[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    out[(size_t)t * C + c] = from_float<T>(0.f);
    return;
  }
  const int at = t - q_start[b];  // place of the token in its portion
  const float ib = in_bias ? in_bias[c] : 0.f;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j) {
    const int back = K - 1 - j;
    float v;
    if (at - back >= 0)
      v = to_float(x[(size_t)(t - back) * ldx + c]) + ib;
    else
      v = state[((size_t)slot * (K - 1) + (K - 1 + at - back)) * C + c];
    acc = fmaf(w[(size_t)c * K + j], v, acc);
  }
  out[(size_t)t * C + c] = from_float<T>(activate(acc, act));
}

// grid (requests, channel chunks): the last K - 1 inputs of each request, from the portion and, where the
// portion is shorter than that, from the old state (moved up in place, oldest first).
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ in_bias,
                                  float* __restrict__ state, const int* __restrict__ q_start,
                                  const int* __restrict__ slot_ids, int C, int K, int num_slots) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = slot_ids[b];
  if (c >= C || slot < 0 || slot >= num_slots) return;
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  const float ib = in_bias ? in_bias[c] : 0.f;
  float* st = state + (size_t)slot * (K - 1) * C + c;
  for (int i = 0; i < K - 1; ++i) {
    const int p = n - (K - 1) + i;  // place in the portion of the input that entry i will hold
    st[(size_t)i * C] = p >= 0 ? to_float(x[(size_t)(t0 + p) * ldx + c]) + ib : st[(size_t)(i + n) * C];
  }
}

// ---------------------------------------------------------------- block-diagonal product
// u: [T, C], C = nb * bw; w: [nb, rows, bw] (rows = the stacked output rows of a block); out: float32
// [nb, T, rows].  One warp per output row of a block: the row of w stays in registers while the warp walks
// over the tokens, so the weight is read once per launch; a (token, row) sum is lane-strided products and a
// shuffle reduction, the same for every number of tokens.  For few tokens and for the float32 path; many
// tokens in bfloat16 go to the library's batched product.
constexpr int BD_WARPS = 8;
constexpr int BD_MAX_PER_LANE = 32;  // bw up to 1024

template <typename T>
__global__ void __launch_bounds__(BD_WARPS * 32)
block_diag_kernel(const T* __restrict__ u, const T* __restrict__ w, float* __restrict__ out, int Ttot, int C, int nb,
                  int bw, int rows) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * BD_WARPS + (threadIdx.x >> 5);
  if (unit >= nb * rows) return;
  const int blk = unit / rows, r = unit % rows;
  const T* wr = w + ((size_t)blk * rows + r) * bw;
  float wv[BD_MAX_PER_LANE];
#pragma unroll
  for (int k = 0; k < BD_MAX_PER_LANE; ++k) {
    const int e = lane + 32 * k;
    wv[k] = e < bw ? to_float(wr[e]) : 0.f;
  }
  for (int t = 0; t < Ttot; ++t) {
    const T* ur = u + (size_t)t * C + (size_t)blk * bw;
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < BD_MAX_PER_LANE; ++k) {
      const int e = lane + 32 * k;
      if (e < bw) dot = fmaf(wv[k], to_float(ur[e]), dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) out[((size_t)blk * Ttot + t) * rows + r] = dot;
  }
}

// ---------------------------------------------------------------- gated linear recurrence (RG-LRU)
// grid (requests, channel chunks), one thread per channel, tokens one after the other.
// proj: [T, ld_proj], the y branch's pre-activation at column y_col; u: [T, C]; gates: float32 [nb, T, 2 bw]
// (per block the recurrence gate's rows, then the input gate's); state: float32 [slots, C].
template <typename T>
__global__ void rglru_scan_kernel(const T* __restrict__ proj, int ld_proj, int y_col, const float* __restrict__ y_bias,
                                  const T* __restrict__ u, const float* __restrict__ gates,
                                  const float* __restrict__ ra_bias, const float* __restrict__ ri_bias,
                                  const float* __restrict__ lam, float decay, float* __restrict__ state,
                                  const int* __restrict__ q_start, const int* __restrict__ slot_ids,
                                  T* __restrict__ out, int Ttot, int C, int bw, int num_slots, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int slot = slot_ids[b];
  const int t0 = q_start[b], t1 = q_start[b + 1];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    for (int t = t0; t < t1; ++t) out[(size_t)t * C + c] = from_float<T>(0.f);
    return;
  }
  const int blk = c / bw, j = c - blk * bw;
  const float rate = -decay * softplus_f(lam[c]);
  const float rb = ra_bias[c], ib = ri_bias[c], yb = y_bias ? y_bias[c] : 0.f;
  float S = state[(size_t)slot * C + c];
  const float* g = gates + ((size_t)blk * Ttot + t0) * 2 * bw;
  for (int t = t0; t < t1; ++t, g += 2 * bw) {
    const float r = sigmoid_f(g[j] + rb);
    const float i = sigmoid_f(g[bw + j] + ib);
    const float log_a = rate * r;
    const float a = expf(log_a);
    const float m = sqrtf(-expm1f(2.f * log_a));  // sqrt(1 - a^2) without the cancellation near a = 1
    S = fmaf(a, S, m * i * to_float(u[(size_t)t * C + c]));
    const float y = gelu_tanh_f(to_float(proj[(size_t)t * ld_proj + y_col + c]) + yb);
    out[(size_t)t * C + c] = from_float<T>(S * y);
  }
  state[(size_t)slot * C + c] = S;
}

// ---------------------------------------------------------------- selective scan (Mamba)
// grid (requests, channel chunks), one thread per channel with its N state values in registers.
// xc: [T, I] (after convolution and activation); proj: [T, ld_proj] with z at column z_col; bc: float32
// [T, 2 N] (B then C); dt: float32 [T, I] before bias and softplus; state: float32 [slots, N, I].
template <typename T, int NMAX>
__global__ void selective_scan_kernel(const T* __restrict__ xc, const T* __restrict__ proj, int ld_proj, int z_col,
                                      const float* __restrict__ bc, const float* __restrict__ dt,
                                      const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                      const float* __restrict__ Dp, float* __restrict__ state,
                                      const int* __restrict__ q_start, const int* __restrict__ slot_ids,
                                      T* __restrict__ out, int I, int N, int num_slots, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= I) return;
  const int slot = slot_ids[b];
  const int t0 = q_start[b], t1 = q_start[b + 1];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    for (int t = t0; t < t1; ++t) out[(size_t)t * I + c] = from_float<T>(0.f);
    return;
  }
  float A[NMAX], S[NMAX];
  float* st = state + (size_t)slot * N * I + c;
#pragma unroll
  for (int n = 0; n < NMAX; ++n) {
    A[n] = n < N ? -expf(A_log[(size_t)c * N + n]) : 0.f;
    S[n] = n < N ? st[(size_t)n * I] : 0.f;
  }
  const float db = dt_bias[c], dskip = Dp[c];
  for (int t = t0; t < t1; ++t) {
    const float step = softplus_f(dt[(size_t)t * I + c] + db);
    const float x = to_float(xc[(size_t)t * I + c]);
    const float sx = step * x;
    const float* Bt = bc + (size_t)t * 2 * N;
    const float* Ct = Bt + N;
    float y = 0.f;
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      if (n < N) {
        S[n] = fmaf(expf(step * A[n]), S[n], sx * Bt[n]);
        y = fmaf(S[n], Ct[n], y);
      }
    }
    y = fmaf(dskip, x, y);
    const float z = to_float(proj[(size_t)t * ld_proj + z_col + c]);
    out[(size_t)t * I + c] = from_float<T>(y * silu_f(z));
  }
#pragma unroll
  for (int n = 0; n < NMAX; ++n)
    if (n < N) st[(size_t)n * I] = S[n];
}

template <typename T>
static int selective_scan_launch(const void* xc, const void* proj, int ld_proj, int z_col, const float* bc, const float* dt,
                                 const float* dt_bias, const float* A_log, const float* Dp, float* state,
                                 const int* q_start, const int* slot_ids, void* out, int B, int I, int N, int num_slots,
                                 int* status, cudaStream_t stream) {
  const int threads = 64;
  dim3 grid(B, (I + threads - 1) / threads);
#define Q3_SS(NM)                                                                                                  \
  q3::launch(selective_scan_kernel<T, NM>, grid, dim3(threads), 0, stream, (const T*)xc, (const T*)proj, ld_proj, z_col, \
             bc, dt, dt_bias, A_log, Dp, state, q_start, slot_ids, (T*)out, I, N, num_slots, status)
  if (N <= 8) Q3_SS(8);
  else if (N <= 16) Q3_SS(16);
  else if (N <= 32) Q3_SS(32);
  else if (N <= 64) Q3_SS(64);
  else if (N <= 128) Q3_SS(128);
  else return Q3_ERR_SIZE;
#undef Q3_SS
  return launch_status();
}

}  // namespace q3

#define Q3_BY_DTYPE(dtype, CALL)                 \
  if ((dtype) == Q3_F32) { using E = float; CALL; }  \
  else if ((dtype) == Q3_BF16) { using E = __nv_bfloat16; CALL; } \
  else return Q3_ERR_DTYPE;

// out[t] = x[t] + (x[t - 1] - x[t]) * mu in `dtype`; x: float32 [T, W]; state: float32 [num_slots, W].
extern "C" int q3_token_shift(const float* x, const float* mu, float* state, const int* q_start, const int* tok_seq,
                              const int* slot_ids, void* out, int dtype, int T, int W, int num_slots, int* status,
                              cudaStream_t stream) {
  if (T <= 0 || W <= 0) return 0;
  int threads = ((W + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  Q3_BY_DTYPE(dtype, q3::launch(q3::token_shift_kernel<E>, dim3(T), dim3(threads), 0, stream, x, mu, state, q_start, tok_seq,
                                slot_ids, (E*)out, W, num_slots, status))
  return q3::launch_status();
}

// The convolution of a step's tokens, then the state's renewal (two launches).  x: [T, ldx] in `dtype`, the
// channels at x (the caller offsets the pointer); w: float32 [C, K]; state: float32 [num_slots, K - 1, C].
extern "C" int q3_causal_conv(const void* x, int ldx, const float* in_bias, const float* w, const float* bias, float* state,
                              const int* q_start, const int* tok_seq, const int* slot_ids, void* out, int dtype, int T,
                              int B, int C, int K, int act, int num_slots, int* status, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  if (K <= 0 || B <= 0 || act < Q3_ACT_SILU || act > Q3_ACT_NONE) return Q3_ERR_SIZE;
  const int threads = 128;
  dim3 grid(T, (C + threads - 1) / threads), sgrid(B, (C + threads - 1) / threads);
  if (grid.y > 65535) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, {
    q3::launch(q3::causal_conv_kernel<E>, grid, dim3(threads), 0, stream, (const E*)x, ldx, in_bias, w, bias,
               (const float*)state, q_start, tok_seq, slot_ids, (E*)out, C, K, act, num_slots, status);
    if (K > 1)
      q3::launch(q3::conv_state_kernel<E>, sgrid, dim3(threads), 0, stream, (const E*)x, ldx, in_bias, state, q_start,
                 slot_ids, C, K, num_slots);
  })
  return q3::launch_status();
}

// out[blk, t, r] = sum_e w[blk, r, e] * u[t, blk * bw + e]; u and w in `dtype`, out float32.
extern "C" int q3_block_diag(const void* u, const void* w, float* out, int dtype, int T, int nb, int bw, int rows,
                             cudaStream_t stream) {
  if (T <= 0 || nb <= 0 || rows <= 0) return 0;
  if (bw <= 0 || bw > 32 * q3::BD_MAX_PER_LANE) return Q3_ERR_SIZE;
  const int units = nb * rows;
  dim3 grid((units + q3::BD_WARPS - 1) / q3::BD_WARPS);
  Q3_BY_DTYPE(dtype, q3::launch(q3::block_diag_kernel<E>, grid, dim3(q3::BD_WARPS * 32), 0, stream, (const E*)u, (const E*)w,
                                out, T, nb * bw, nb, bw, rows))
  return q3::launch_status();
}

extern "C" int q3_rglru_scan(const void* proj, int ld_proj, int y_col, const float* y_bias, const void* u, const float* gates,
                             const float* ra_bias, const float* ri_bias, const float* lam, float decay, float* state,
                             const int* q_start, const int* slot_ids, void* out, int dtype, int T, int B, int C, int bw,
                             int num_slots, int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0 || C <= 0) return 0;
  if (bw <= 0 || C % bw) return Q3_ERR_SIZE;
  const int threads = 64;
  dim3 grid(B, (C + threads - 1) / threads);
  if (grid.y > 65535) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::rglru_scan_kernel<E>, grid, dim3(threads), 0, stream, (const E*)proj, ld_proj, y_col, y_bias,
                                (const E*)u, gates, ra_bias, ri_bias, lam, decay, state, q_start, slot_ids, (E*)out, T, C, bw,
                                num_slots, status))
  return q3::launch_status();
}

// State sizes up to 128 (kept in registers).
extern "C" int q3_selective_scan(const void* xc, const void* proj, int ld_proj, int z_col, const float* bc, const float* dt,
                                 const float* dt_bias, const float* A_log, const float* Dp, float* state,
                                 const int* q_start, const int* slot_ids, void* out, int dtype, int T, int B, int I, int N,
                                 int num_slots, int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0 || I <= 0) return 0;
  if (N <= 0) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, return q3::selective_scan_launch<E>(xc, proj, ld_proj, z_col, bc, dt, dt_bias, A_log, Dp, state, q_start,
                                                         slot_ids, out, B, I, N, num_slots, status, stream))
}
