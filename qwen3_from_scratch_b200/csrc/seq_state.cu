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

__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------- token shift
// One block per token.  The block of a request's first token of the step reads the state (the x of the
// token before) and, element by element after reading it, stores the portion's last x there.
// Four features per thread with 16-byte loads (W a multiple of 4, rows 16-byte aligned); otherwise as below.
template <typename T>
__global__ void token_shift_vec4_kernel(const float* __restrict__ x, const float* __restrict__ mu, float* __restrict__ state,
                                        const int* __restrict__ q_start, const int* __restrict__ tok_seq,
                                        const int* __restrict__ slot_ids, T* __restrict__ out, int W, int num_slots,
                                        int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  const int slot = slot_ids[b];
  const bool live = slot >= 0 && slot < num_slots;
  if (!live && threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
  const bool first = t == q_start[b];
  const float* cur = x + (size_t)t * W;
  const float* prev = first ? (live ? state + (size_t)slot * W : nullptr) : cur - W;
  const float* last = x + (size_t)(q_start[b + 1] - 1) * W;
  T* o = out + (size_t)t * W;
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    const float4 c = *reinterpret_cast<const float4*>(cur + i);
    const float4 m = *reinterpret_cast<const float4*>(mu + i);
    const float4 p = prev ? *reinterpret_cast<const float4*>(prev + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float r[4] = {c.x + (p.x - c.x) * m.x, c.y + (p.y - c.y) * m.y, c.z + (p.z - c.z) * m.z, c.w + (p.w - c.w) * m.w};
    if (!live) {
      for (int k = 0; k < 4; ++k) o[i + k] = from_float<T>(0.f);
      continue;
    }
    if (sizeof(T) == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(o + i) = pk;
    } else {
      *reinterpret_cast<float4*>(o + i) = make_float4(r[0], r[1], r[2], r[3]);
    }
    // the element's old state has been read by this thread and by nobody else: it may be renewed now
    if (first) *reinterpret_cast<float4*>(state + (size_t)slot * W + i) = *reinterpret_cast<const float4*>(last + i);
  }
}

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
// float32, entry K - 2 the newest.  The state of a longer portion is only read here (its first K - 1 tokens read
// it from several blocks); conv_state_kernel renews it afterwards.
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ in_bias,
                                   const float* __restrict__ w, const float* __restrict__ bias,
                                   float* __restrict__ state, const int* __restrict__ q_start,
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
  const bool single = q_start[b + 1] - q_start[b] == 1;
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
    // a portion of one token: nobody else reads this channel's tail, so it moves up here (what tap j read becomes
    // entry j - 1) and the renewing kernel leaves the request alone
    if (single && j > 0) state[((size_t)slot * (K - 1) + j - 1) * C + c] = v;
  }
  out[(size_t)t * C + c] = from_float<T>(activate(acc, act));
}

// bfloat16, C a multiple of 8, K up to CONV_KMAX: a thread takes eight channels (16-byte loads and stores) and a run
// of CONV_RUN tokens, keeps the taps and the window of the last K - 1 inputs in registers and slides the window from
// token to token; at a request's first token of the step the window is refilled from the state.  All of the run's
// inputs are asked for before the first is used, so that a thread has CONV_RUN loads in flight.  The state is
// only read here, also for a portion of one token (conv_state_kernel renews every request's afterwards).
constexpr int CONV_KMAX = 4, CONV_RUN = 8;  // the kernel is compiled for each number of taps up to CONV_KMAX

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    f[2 * k] = __uint_as_float(w[k] << 16);
    f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
  }
}

template <int K>
__global__ void causal_conv_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const float* __restrict__ in_bias,
                                          const float* __restrict__ w, const float* __restrict__ bias,
                                          const float* __restrict__ state, const int* __restrict__ q_start,
                                          const int* __restrict__ tok_seq, const int* __restrict__ slot_ids,
                                          __nv_bfloat16* __restrict__ out, int Ttot, int C, int act, int num_slots,
                                          int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int t0 = blockIdx.x * CONV_RUN, t1 = min(Ttot, t0 + CONV_RUN);
  float taps[K][8], ib[8], cb[8], win[K > 1 ? K - 1 : 1][8];  // win[0] the oldest of the K - 1 inputs before the token
  {
    // the thread's 8 K taps lie side by side in w ([C, K]); they and the biases come in 16-byte loads (c is a
    // multiple of 8 and the launcher has checked the pointers), not one by one: a thread has only CONV_RUN tokens
    // to spread this preamble over
    float flat[8 * K];
#pragma unroll
    for (int i = 0; i < 2 * K; ++i) {
      const float4 f = reinterpret_cast<const float4*>(w + (size_t)c * K)[i];
      flat[4 * i] = f.x; flat[4 * i + 1] = f.y; flat[4 * i + 2] = f.z; flat[4 * i + 3] = f.w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (int j = 0; j < K; ++j) taps[j][e] = flat[e * K + j];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float4 a = in_bias ? reinterpret_cast<const float4*>(in_bias + c)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 b = bias ? reinterpret_cast<const float4*>(bias + c)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      ib[4 * i] = a.x; ib[4 * i + 1] = a.y; ib[4 * i + 2] = a.z; ib[4 * i + 3] = a.w;
      cb[4 * i] = b.x; cb[4 * i + 1] = b.y; cb[4 * i + 2] = b.z; cb[4 * i + 3] = b.w;
    }
  }
  // entry i of the window before token t, place `at` in its portion: the input `K - 1 - i` tokens back
  auto fill = [&](int t, int at, int slot) {
#pragma unroll
    for (int i = 0; i < K - 1; ++i) {
      const int back = K - 1 - i;
      if (at - back >= 0) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(x + (size_t)(t - back) * ldx + c), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) win[i][e] = f[e] + ib[e];
      } else {
        const float4* st = reinterpret_cast<const float4*>(state + ((size_t)(slot < 0 ? 0 : slot) * (K - 1) + (K - 1 + at - back)) * C + c);
        const float4 lo = slot >= 0 ? st[0] : make_float4(0.f, 0.f, 0.f, 0.f), hi = slot >= 0 ? st[1] : lo;
        win[i][0] = lo.x; win[i][1] = lo.y; win[i][2] = lo.z; win[i][3] = lo.w;
        win[i][4] = hi.x; win[i][5] = hi.y; win[i][6] = hi.z; win[i][7] = hi.w;
      }
    }
  };
  uint4 raw[CONV_RUN];
  int seq[CONV_RUN];
#pragma unroll
  for (int i = 0; i < CONV_RUN; ++i) {
    const int t = t0 + i;
    raw[i] = t < t1 ? *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + c) : make_uint4(0, 0, 0, 0);
    seq[i] = t < t1 ? tok_seq[t] : 0;
  }
#pragma unroll
  for (int i = 0; i < CONV_RUN; ++i) {
    const int t = t0 + i;
    if (t >= t1) break;
    const int b = seq[i];
    const int at = t - q_start[b];
    if (i == 0 || at == 0) {
      int slot = slot_ids[b];
      if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
        slot = -1;
      }
      fill(t, at, slot);
    }
    float v[8], acc[8];
    unpack8(raw[i], v);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[e] += ib[e];
      acc[e] = cb[e];
#pragma unroll
      for (int j = 0; j < K - 1; ++j) acc[e] = fmaf(taps[j][e], win[j][e], acc[e]);
      acc[e] = fmaf(taps[K - 1][e], v[e], acc[e]);
    }
    // the result is rounded to bfloat16: the SiLU takes the hardware's exponential and reciprocal
    if (act == Q3_ACT_SILU) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = acc[e] * __fdividef(1.0f, 1.0f + __expf(-acc[e]));
    } else if (act != Q3_ACT_NONE) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = activate(acc[e], act);
    }
    uint4 pk;
    pk.x = pack_pair(acc[0], acc[1]);
    pk.y = pack_pair(acc[2], acc[3]);
    pk.z = pack_pair(acc[4], acc[5]);
    pk.w = pack_pair(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (size_t)t * C + c) = pk;
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
#pragma unroll
      for (int e = 0; e < 8; ++e) win[j][e] = (j + 1 < K - 1) ? win[j + 1 < K - 1 ? j + 1 : j][e] : v[e];
    }
  }
}

// grid (requests, channel chunks): the last K - 1 inputs of each request, from the portion and, where the
// portion is shorter than that, from the old state (moved up in place, oldest first).
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ in_bias,
                                  float* __restrict__ state, const int* __restrict__ q_start,
                                  const int* __restrict__ slot_ids, int C, int K, int num_slots, int singles_too) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = slot_ids[b];
  if (c >= C || slot < 0 || slot >= num_slots) return;
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  if (n == 1 && !singles_too) return;  // the plain convolution kernel has moved a single token's tail itself
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
constexpr int BD_MAX_PER_LANE = 32;  // rows of up to 1024 values stay in registers

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
  if (bw > 32 * BD_MAX_PER_LANE) {  // a block too wide for the registers: its row is read again for every token
    for (int t = 0; t < Ttot; ++t) {
      const T* ur = u + (size_t)t * C + (size_t)blk * bw;
      float dot = 0.f;
      for (int e = lane; e < bw; e += 32) dot = fmaf(to_float(wr[e]), to_float(ur[e]), dot);
      dot = warp_sum(dot);
      if (lane == 0) out[((size_t)blk * Ttot + t) * rows + r] = dot;
    }
    return;
  }
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

// a S + b for a = exp(log_a) in the float32 run.  A decay near 1 carries a state over thousands of tokens, and
// expf's error of an ulp of 1 at every step would add up along the way; there the update is S + (b - (1 - a) S)
// with 1 - a = -expm1(log_a), whose error is relative to 1 - a.  A fast decay (a below one half) keeps the
// plain form, in which nothing of the size of the old state is added and taken away again.
__device__ __forceinline__ float slow_decay_update(float log_a, float S, float b) {
  return log_a > -0.6931472f ? S + fmaf(expm1f(log_a), S, b) : fmaf(expf(log_a), S, b);
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
    const float m = sqrtf(-expm1f(2.f * log_a));  // sqrt(1 - a^2) without the cancellation near a = 1
    const float b = m * i * to_float(u[(size_t)t * C + c]);
    if (sizeof(T) == 4) {
      S = slow_decay_update(log_a, S, b);
    } else {
      S = fmaf(expf(log_a), S, b);
    }
    const float y = gelu_tanh_f(to_float(proj[(size_t)t * ld_proj + y_col + c]) + yb);
    out[(size_t)t * C + c] = from_float<T>(S * y);
  }
  state[(size_t)slot * C + c] = S;
}

// A token's N values of B (or C) into registers, four at a time where N and the row allow 16-byte loads.
template <int NMAX>
__device__ __forceinline__ void load_row(const float* __restrict__ row, int N, float (&v)[NMAX]) {
  if (NMAX >= 4 && N % 4 == 0 && ((uintptr_t)row & 15) == 0) {
#pragma unroll
    for (int n4 = 0; n4 < NMAX / 4; ++n4) {
      if (4 * n4 < N) {
        const float4 f = reinterpret_cast<const float4*>(row)[n4];
        v[4 * n4] = f.x; v[4 * n4 + 1] = f.y; v[4 * n4 + 2] = f.z; v[4 * n4 + 3] = f.w;
      }
    }
  } else {
#pragma unroll
    for (int n = 0; n < NMAX; ++n)
      if (n < N) v[n] = row[n];
  }
}

// exp(step * A) with A = -exp(A_log): the float32 run evaluates it as written; the bfloat16 run keeps A in units of
// the base-2 exponential and takes exp2f, a shorter sequence whose error (2 ulp) is far below that run's roundings.
template <typename T> __device__ __forceinline__ float decay_rate(float a_log) {
  return sizeof(T) == 4 ? -expf(a_log) : -expf(a_log) * 1.4426950408889634f;
}
template <typename T> __device__ __forceinline__ float decay(float step, float rate) {
  if (sizeof(T) == 4) return expf(step * rate);
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(step * rate));
  return y;
}
// softplus and SiLU of the scans: as written in the float32 run; in the bfloat16 run by the hardware's base-2
// exponential, logarithm and reciprocal (relative error about 2^-21, still float32 arithmetic), because the special
// function unit, which also serves the library forms' slow paths, is what bounds these kernels.
template <typename T> __device__ __forceinline__ float scan_softplus(float x) {
  if (sizeof(T) == 4) return softplus_f(x);
  return fmaxf(x, 0.f) + __logf(1.0f + __expf(-fabsf(x)));
}
template <typename T> __device__ __forceinline__ float scan_silu(float z) {
  if (sizeof(T) == 4) return silu_f(z);
  return z * __fdividef(1.0f, 1.0f + __expf(-z));
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
    A[n] = n < N ? decay_rate<T>(A_log[(size_t)c * N + n]) : 0.f;
    S[n] = n < N ? st[(size_t)n * I] : 0.f;
  }
  const float db = dt_bias[c], dskip = Dp[c];
  for (int t = t0; t < t1; ++t) {
    const float step = scan_softplus<T>(dt[(size_t)t * I + c] + db);
    const float x = to_float(xc[(size_t)t * I + c]);
    const float sx = step * x;
    float Bt[NMAX], Ct[NMAX];
    load_row<NMAX>(bc + (size_t)t * 2 * N, N, Bt);
    load_row<NMAX>(bc + (size_t)t * 2 * N + N, N, Ct);
    float y = 0.f;
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      if (n < N) {
        if (sizeof(T) == 4)  // see slow_decay_update
          S[n] = slow_decay_update(step * A[n], S[n], sx * Bt[n]);
        else
          S[n] = fmaf(decay<T>(step, A[n]), S[n], sx * Bt[n]);
        y = fmaf(S[n], Ct[n], y);
      }
    }
    y = fmaf(dskip, x, y);
    const float z = to_float(proj[(size_t)t * ld_proj + z_col + c]);
    out[(size_t)t * I + c] = from_float<T>(y * scan_silu<T>(z));
  }
#pragma unroll
  for (int n = 0; n < NMAX; ++n)
    if (n < N) st[(size_t)n * I] = S[n];
}

// ---------------------------------------------------------------- the same recurrences over chunks of a portion
// A thread per channel walks a whole portion alone, which leaves most of the GPU idle when a long portion of a
// single request runs: the portion is then cut into chunks of SCAN_CHUNK tokens that run side by side in three
// launches.  Both recurrences are linear in the state, S_t = a_t S_{t-1} + b_t, so a chunk is summarised by the
// product P of its a_t and the state V that it reaches from zero; then, chunk after chunk, S_in(j + 1) =
// P_j S_in(j) + V_j (a loop of portion / SCAN_CHUNK steps), and each chunk is walked again from its S_in.
// Chunk j of request b is filed at scratch index q_start[b] / SCAN_CHUNK + b + j, which never collides: a
// request of n tokens has at most n / SCAN_CHUNK + 1 chunks.  The sums differ from the single walk's by float32
// rounding; the float32 run keeps the single walk, so that its bits do not depend on the cut.  The chunked kernels
// are the bfloat16 run's alone and take the hardware's special functions (see rglru_coeffs, decay, scan_softplus).
constexpr int SCAN_CHUNK = 64;

// The bfloat16 run's forms of the RG-LRU's functions: the hardware's exponential, reciprocal and tanh (float32
// arithmetic, relative error near 2^-21; 1 - a^2 as written, whose rounding only matters where the term vanishes).
__device__ __forceinline__ float fast_sigmoid_f(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float fast_gelu_tanh_f(float z) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return 0.5f * z * (1.0f + t);
}

__device__ __forceinline__ void rglru_coeffs(float g_r, float g_i, float rb, float ib, float rate, float u, float& a,
                                             float& b) {
  const float r = fast_sigmoid_f(g_r + rb), i = fast_sigmoid_f(g_i + ib);
  a = __expf(rate * r);
  b = sqrtf(fmaxf(1.0f - a * a, 0.f)) * i * u;
}

// PASS 1: the chunk's product and zero-start state into scratch [chunk][2][C].  PASS 3: the walk from the chunk's
// incoming state (left in scratch [chunk][0][C] by the carry kernel), writing the output.
template <typename T, int PASS>
__global__ void rglru_chunk_kernel(const T* __restrict__ proj, int ld_proj, int y_col, const float* __restrict__ y_bias,
                                   const T* __restrict__ u, const float* __restrict__ gates,
                                   const float* __restrict__ ra_bias, const float* __restrict__ ri_bias,
                                   const float* __restrict__ lam, float decay, float* __restrict__ scratch,
                                   const int* __restrict__ q_start, T* __restrict__ out, int Ttot, int C, int bw) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, j = blockIdx.y;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  const int t0 = q_start[b] + j * SCAN_CHUNK, end = q_start[b + 1];
  if (c >= C || t0 >= end) return;
  const int t1 = min(end, t0 + SCAN_CHUNK);
  float* sc = scratch + ((size_t)(q_start[b] / SCAN_CHUNK + b + j) * 2) * C + c;
  const int blk = c / bw, jj = c - blk * bw;
  const float rate = -decay * softplus_f(lam[c]);
  const float rb = ra_bias[c], ib = ri_bias[c], yb = (PASS == 3 && y_bias) ? y_bias[c] : 0.f;
  float S = PASS == 3 ? sc[0] : 0.f, P = 1.f;
  const float* g = gates + ((size_t)blk * Ttot + t0) * 2 * bw;
#pragma unroll 4
  for (int t = t0; t < t1; ++t, g += 2 * bw) {
    float a, bb;
    rglru_coeffs(g[jj], g[bw + jj], rb, ib, rate, to_float(u[(size_t)t * C + c]), a, bb);
    S = fmaf(a, S, bb);
    if (PASS == 1) P *= a;
    if (PASS == 3) {
      const float y = fast_gelu_tanh_f(to_float(proj[(size_t)t * ld_proj + y_col + c]) + yb);
      out[(size_t)t * C + c] = from_float<T>(S * y);
    }
  }
  if (PASS == 1) {
    sc[0] = P;
    sc[C] = S;
  }
}

// grid (requests, channel chunks): scratch [chunk][0] becomes the chunk's incoming state; the request's state slot
// receives the state after its last chunk.
__global__ void rglru_carry_kernel(float* __restrict__ scratch, float* __restrict__ state, const int* __restrict__ q_start,
                                   const int* __restrict__ slot_ids, int C, int num_slots, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int slot = slot_ids[b];
  const bool live = slot >= 0 && slot < num_slots;
  if (!live && threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
  const int n = q_start[b + 1] - q_start[b];
  const int chunks = (n + SCAN_CHUNK - 1) / SCAN_CHUNK;
  float* sc = scratch + ((size_t)(q_start[b] / SCAN_CHUNK + b) * 2) * C + c;
  float S = live ? state[(size_t)slot * C + c] : 0.f;
  for (int j0 = 0; j0 < chunks; j0 += 8) {  // eight records are asked for together, then walked
    float P[8], V[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const bool in = j0 + k < chunks;
      P[k] = in ? sc[(size_t)(j0 + k) * 2 * C] : 1.f;
      V[k] = in ? sc[(size_t)(j0 + k) * 2 * C + C] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (j0 + k < chunks) sc[(size_t)(j0 + k) * 2 * C] = S;
      S = fmaf(P[k], S, V[k]);
    }
  }
  if (live) state[(size_t)slot * C + c] = S;
}

// Selective scan by chunks.  scratch [chunk][N + 1][I]: PASS 1 leaves the zero-start state per n and, at n = N, the
// chunk's sum of step sizes (the chunk's product of exp(step A[c, n]) is exp(A[c, n] * that sum)); the carry kernel
// turns the N entries into the incoming state; PASS 3 walks the chunk from it and writes the output.
// FULL: N == NMAX, which spares the kernel its question "n < N" at every state of every token.
template <typename T, int NMAX, int PASS, bool FULL>
__global__ void __launch_bounds__(64, NMAX <= 16 ? 16 : 1)  // small states: 64 registers, so that an SM holds 32 warps
selective_chunk_kernel(const T* __restrict__ xc, const T* __restrict__ proj, int ld_proj, int z_col,
                                       const float* __restrict__ bc, const float* __restrict__ dt,
                                       const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                       const float* __restrict__ Dp, float* __restrict__ scratch,
                                       const int* __restrict__ q_start, T* __restrict__ out, int I, int N) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, j = blockIdx.y;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  const int t0 = q_start[b] + j * SCAN_CHUNK, end = q_start[b + 1];
  if (c >= I || t0 >= end) return;
  const int t1 = min(end, t0 + SCAN_CHUNK);
  float* sc = scratch + ((size_t)(q_start[b] / SCAN_CHUNK + b + j) * (N + 1)) * I + c;
  float A[NMAX], S[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) {
    A[n] = (FULL || n < N) ? decay_rate<T>(A_log[(size_t)c * N + n]) : 0.f;
    S[n] = (PASS == 3 && (FULL || n < N)) ? sc[(size_t)n * I] : 0.f;
  }
  const float db = dt_bias[c], dskip = PASS == 3 ? Dp[c] : 0.f;
  float sum_step = 0.f;
  // a token's operands are asked for one token ahead, so that their way from memory is covered by the arithmetic of
  // the token before (the blocks are small and few: nothing else would hide it)
  float dt_n = dt[(size_t)t0 * I + c], x_n = to_float(xc[(size_t)t0 * I + c]);
  float z_n = PASS == 3 ? to_float(proj[(size_t)t0 * ld_proj + z_col + c]) : 0.f;
  float B_n[NMAX], C_n[NMAX];
  load_row<NMAX>(bc + (size_t)t0 * 2 * N, N, B_n);
  if (PASS == 3) load_row<NMAX>(bc + (size_t)t0 * 2 * N + N, N, C_n);
  for (int t = t0; t < t1; ++t) {
    const float dt_c = dt_n, x = x_n, z = z_n;
    float Bt[NMAX], Ct[NMAX];
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      Bt[n] = B_n[n];
      if (PASS == 3) Ct[n] = C_n[n];
    }
    if (t + 1 < t1) {
      dt_n = dt[(size_t)(t + 1) * I + c];
      x_n = to_float(xc[(size_t)(t + 1) * I + c]);
      if (PASS == 3) z_n = to_float(proj[(size_t)(t + 1) * ld_proj + z_col + c]);
      load_row<NMAX>(bc + (size_t)(t + 1) * 2 * N, N, B_n);
      if (PASS == 3) load_row<NMAX>(bc + (size_t)(t + 1) * 2 * N + N, N, C_n);
    }
    const float step = scan_softplus<T>(dt_c + db);
    const float sx = step * x;
    float y = 0.f;
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      if (FULL || n < N) {
        S[n] = fmaf(decay<T>(step, A[n]), S[n], sx * Bt[n]);
        if (PASS == 3) y = fmaf(S[n], Ct[n], y);
      }
    }
    if (PASS == 1) sum_step += step;
    if (PASS == 3) {
      y = fmaf(dskip, x, y);
      out[(size_t)t * I + c] = from_float<T>(y * scan_silu<T>(z));
    }
  }
  if (PASS == 1) {
#pragma unroll
    for (int n = 0; n < NMAX; ++n)
      if (FULL || n < N) sc[(size_t)n * I] = S[n];
    sc[(size_t)N * I] = sum_step;
  }
}

// grid (requests, channel chunks, N): one thread per (channel, n).
__global__ void selective_carry_kernel(float* __restrict__ scratch, const float* __restrict__ A_log,
                                       float* __restrict__ state, const int* __restrict__ q_start,
                                       const int* __restrict__ slot_ids, int I, int N, int num_slots, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, n = blockIdx.z;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= I) return;
  const int slot = slot_ids[b];
  const bool live = slot >= 0 && slot < num_slots;
  if (!live && threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
  const int len = q_start[b + 1] - q_start[b];
  const int chunks = (len + SCAN_CHUNK - 1) / SCAN_CHUNK;
  const float A = -expf(A_log[(size_t)c * N + n]);
  float* sc = scratch + ((size_t)(q_start[b] / SCAN_CHUNK + b) * (N + 1)) * I + c;
  float* st = state + ((size_t)slot * N + n) * I + c;
  float S = live ? *st : 0.f;
  const size_t pitch = (size_t)(N + 1) * I;
  for (int j0 = 0; j0 < chunks; j0 += 8) {  // eight records are asked for together, then walked
    float P[8], V[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const bool in = j0 + k < chunks;
      V[k] = in ? sc[(j0 + k) * pitch + (size_t)n * I] : 0.f;
      P[k] = in ? sc[(j0 + k) * pitch + (size_t)N * I] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (j0 + k < chunks) sc[(j0 + k) * pitch + (size_t)n * I] = S;
      S = fmaf(expf(A * P[k]), S, V[k]);
    }
  }
  if (live) *st = S;
}

template <typename T>
static int selective_chunked_launch(const void* xc, const void* proj, int ld_proj, int z_col, const float* bc,
                                    const float* dt, const float* dt_bias, const float* A_log, const float* Dp,
                                    float* state, float* scratch, const int* q_start, const int* slot_ids, void* out,
                                    int B, int max_q_len, int I, int N, int num_slots, int* status, cudaStream_t stream) {
  const int threads = 64;
  const int chunks = (max_q_len + SCAN_CHUNK - 1) / SCAN_CHUNK;
  dim3 grid(B, chunks, (I + threads - 1) / threads), cgrid(B, (I + threads - 1) / threads, N);
  if (chunks > 65535 || grid.z > 65535 || N > 65535) return Q3_ERR_SIZE;
#define Q3_SC_GO(NM, FULL)                                                                                           \
  do {                                                                                                               \
    q3::launch(selective_chunk_kernel<T, NM, 1, FULL>, grid, dim3(threads), 0, stream, (const T*)xc, (const T*)proj,  \
               ld_proj, z_col, bc, dt, dt_bias, A_log, Dp, scratch, q_start, (T*)out, I, N);                          \
    q3::launch(selective_carry_kernel, cgrid, dim3(threads), 0, stream, scratch, A_log, state, q_start, slot_ids, I, N, \
               num_slots, status);                                                                                   \
    q3::launch(selective_chunk_kernel<T, NM, 3, FULL>, grid, dim3(threads), 0, stream, (const T*)xc, (const T*)proj,  \
               ld_proj, z_col, bc, dt, dt_bias, A_log, Dp, scratch, q_start, (T*)out, I, N);                          \
  } while (0)
#define Q3_SC(NM)              \
  do {                         \
    if (N == NM) Q3_SC_GO(NM, true); \
    else Q3_SC_GO(NM, false);  \
  } while (0)
  if (N <= 8) Q3_SC(8);
  else if (N <= 16) Q3_SC(16);
  else if (N <= 32) Q3_SC(32);
  else if (N <= 64) Q3_SC(64);
  else if (N <= 128) Q3_SC(128);
  else return Q3_ERR_SIZE;
#undef Q3_SC_GO
#undef Q3_SC
  return launch_status();
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
  const bool vec = W % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)mu % 16 == 0 && (uintptr_t)state % 16 == 0 &&
                   (uintptr_t)out % 16 == 0;
  int threads = (((vec ? W / 4 : W) + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  if (vec) {
    Q3_BY_DTYPE(dtype, q3::launch(q3::token_shift_vec4_kernel<E>, dim3(T), dim3(threads), 0, stream, x, mu, state, q_start,
                                  tok_seq, slot_ids, (E*)out, W, num_slots, status))
  } else {
    Q3_BY_DTYPE(dtype, q3::launch(q3::token_shift_kernel<E>, dim3(T), dim3(threads), 0, stream, x, mu, state, q_start,
                                  tok_seq, slot_ids, (E*)out, W, num_slots, status))
  }
  return q3::launch_status();
}

// The convolution of a step's tokens, then the state's renewal (a second launch unless every portion is one token).  x: [T, ldx] in `dtype`, the
// channels at x (the caller offsets the pointer); w: float32 [C, K]; state: float32 [num_slots, K - 1, C].
extern "C" int q3_causal_conv(const void* x, int ldx, const float* in_bias, const float* w, const float* bias, float* state,
                              const int* q_start, const int* tok_seq, const int* slot_ids, void* out, int dtype, int T,
                              int B, int C, int K, int act, int num_slots, int* status, cudaStream_t stream) {
  if (T <= 0 || C <= 0) return 0;
  if (K <= 0 || B <= 0 || act < Q3_ACT_SILU || act > Q3_ACT_NONE) return Q3_ERR_SIZE;
  const int threads = 128;
  dim3 grid(T, (C + threads - 1) / threads), sgrid(B, (C + threads - 1) / threads);
  if (grid.y > 65535) return Q3_ERR_SIZE;
  // many tokens in bfloat16: eight channels and a run of tokens per thread; the state is then renewed for every request
  if (dtype == Q3_BF16 && T > B && T >= 4 * q3::CONV_RUN && C % 8 == 0 && K <= q3::CONV_KMAX && ldx % 8 == 0 &&
      (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)state % 16 == 0 &&
      (!in_bias || (uintptr_t)in_bias % 16 == 0) && (!bias || (uintptr_t)bias % 16 == 0)) {
    using bf16 = __nv_bfloat16;
    const int lanes = C / 8;
    const int wide = lanes < 128 ? ((lanes + 31) / 32) * 32 : 128;
    dim3 vgrid((T + q3::CONV_RUN - 1) / q3::CONV_RUN, (lanes + wide - 1) / wide);
#define Q3_CONV(KK)                                                                                                  \
  case KK:                                                                                                           \
    q3::launch(q3::causal_conv_bf16x8_kernel<KK>, vgrid, dim3(wide), 0, stream, (const bf16*)x, ldx, in_bias, w, bias,    \
               (const float*)state, q_start, tok_seq, slot_ids, (bf16*)out, T, C, act, num_slots, status);           \
    break;
    switch (K) { Q3_CONV(1) Q3_CONV(2) Q3_CONV(3) Q3_CONV(4) }
#undef Q3_CONV
    if (K > 1)
      q3::launch(q3::conv_state_kernel<bf16>, sgrid, dim3(threads), 0, stream, (const bf16*)x, ldx, in_bias, state, q_start,
                 slot_ids, C, K, num_slots, 1);
    return q3::launch_status();
  }
  Q3_BY_DTYPE(dtype, {
    q3::launch(q3::causal_conv_kernel<E>, grid, dim3(threads), 0, stream, (const E*)x, ldx, in_bias, w, bias, state,
               q_start, tok_seq, slot_ids, (E*)out, C, K, act, num_slots, status);
    if (K > 1 && T > B)  // T == B: every portion is a single token
      q3::launch(q3::conv_state_kernel<E>, sgrid, dim3(threads), 0, stream, (const E*)x, ldx, in_bias, state, q_start,
                 slot_ids, C, K, num_slots, 0);
  })
  return q3::launch_status();
}

// out[blk, t, r] = sum_e w[blk, r, e] * u[t, blk * bw + e]; u and w in `dtype`, out float32.
extern "C" int q3_block_diag(const void* u, const void* w, float* out, int dtype, int T, int nb, int bw, int rows,
                             cudaStream_t stream) {
  if (T <= 0 || nb <= 0 || rows <= 0) return 0;
  if (bw <= 0) return Q3_ERR_SIZE;
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

// Tokens per chunk of the chunked scans; their scratch holds (tokens / chunk + requests + 1) chunk records.
extern "C" int q3_scan_chunk() { return q3::SCAN_CHUNK; }

// rglru_scan over chunks of the portions (three launches).  scratch: float32, 2 * C per chunk record.
extern "C" int q3_rglru_scan_chunked(const void* proj, int ld_proj, int y_col, const float* y_bias, const void* u,
                                     const float* gates, const float* ra_bias, const float* ri_bias, const float* lam,
                                     float decay, float* state, float* scratch, const int* q_start, const int* slot_ids,
                                     void* out, int dtype, int T, int B, int max_q_len, int C, int bw, int num_slots,
                                     int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0 || C <= 0 || max_q_len <= 0) return 0;
  if (bw <= 0 || C % bw) return Q3_ERR_SIZE;
  const int threads = 64;
  const int chunks = (max_q_len + q3::SCAN_CHUNK - 1) / q3::SCAN_CHUNK;
  dim3 grid(B, chunks, (C + threads - 1) / threads), cgrid(B, (C + threads - 1) / threads);
  if (chunks > 65535 || grid.z > 65535) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, {
    q3::launch(q3::rglru_chunk_kernel<E, 1>, grid, dim3(threads), 0, stream, (const E*)proj, ld_proj, y_col, y_bias,
               (const E*)u, gates, ra_bias, ri_bias, lam, decay, scratch, q_start, (E*)out, T, C, bw);
    q3::launch(q3::rglru_carry_kernel, cgrid, dim3(threads), 0, stream, scratch, state, q_start, slot_ids, C, num_slots,
               status);
    q3::launch(q3::rglru_chunk_kernel<E, 3>, grid, dim3(threads), 0, stream, (const E*)proj, ld_proj, y_col, y_bias,
               (const E*)u, gates, ra_bias, ri_bias, lam, decay, scratch, q_start, (E*)out, T, C, bw);
  })
  return q3::launch_status();
}

// selective_scan over chunks of the portions (three launches).  scratch: float32, (N + 1) * I per chunk record.
extern "C" int q3_selective_scan_chunked(const void* xc, const void* proj, int ld_proj, int z_col, const float* bc,
                                         const float* dt, const float* dt_bias, const float* A_log, const float* Dp,
                                         float* state, float* scratch, const int* q_start, const int* slot_ids, void* out,
                                         int dtype, int T, int B, int max_q_len, int I, int N, int num_slots, int* status,
                                         cudaStream_t stream) {
  if (T <= 0 || B <= 0 || I <= 0 || max_q_len <= 0) return 0;
  if (N <= 0) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, return q3::selective_chunked_launch<E>(xc, proj, ld_proj, z_col, bc, dt, dt_bias, A_log, Dp, state,
                                                            scratch, q_start, slot_ids, out, B, max_q_len, I, N, num_slots,
                                                            status, stream))
}
