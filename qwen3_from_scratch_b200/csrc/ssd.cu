// The state-space recurrence with one scalar decay per head (Mamba-2's), and the gated norm that follows it.
//
//   step = softplus(dt + dt_bias_h);  a = exp(-exp(A_log_h) * step)
//   S_h <- a S_h + step * B_g x_h^T        S_h: [N, P] float32, g = h / (heads / groups)
//   y_h = S_h^T C_g + D_h x_h
//
// x, B and C come from one buffer `xbc` [T, ld] (x: heads * P columns at 0, then groups * N of B, then of C), dt
// from column dt_col of `proj`.  Step sizes, decays and the state are float32 in every run.
//
// ssd_scan: a group of L lanes (a power of two, 16 states each) per head and run of channels walks a request's
// portion token by token; the lanes' parts of y meet in a butterfly of shuffles whose order is the same for every
// cut of a prompt, so the float32 run's bits do not depend on the cut.  The bfloat16 run cuts long portions into
// chunks that run side by side (the recurrence is linear in the state: a chunk is summarised by the product of its
// decays and the state it reaches from zero), and takes the hardware's exponential and logarithm.
// gated_group_norm: y * silu(z), divided by the root mean square of its part (the row is cut into equal parts),
// times a weight.
#include "common.cuh"

namespace q3 {

constexpr int SSD_PER = 16;  // states per lane
constexpr int SSD_CHUNK = 64;  // tokens per chunk of the chunked form

// a S + b with a = exp(log_a): see the note on slowly decaying states in seq_state.cu (the float32 run takes the
// form whose error is relative to 1 - a).
__device__ __forceinline__ float ssd_update(float log_a, float a, float S, float b, bool exact) {
  if (exact && log_a > -0.6931472f) return S + fmaf(expm1f(log_a), S, b);
  return fmaf(a, S, b);
}

// SSD_PER values of row[col ..] as floats; VEC: bfloat16 with col a multiple of 8 and an aligned row (two 16-byte loads).
template <typename T, bool VEC>
__device__ __forceinline__ void ssd_load16(const T* __restrict__ row, int col, int live, float (&v)[SSD_PER]) {
  if constexpr (VEC) {
    if (live <= 0) {  // a lane beyond the last state (the lanes are a power of two): nothing of its own to read
#pragma unroll
      for (int i = 0; i < SSD_PER; ++i) v[i] = 0.f;
      return;
    }
    const uint4 lo = *reinterpret_cast<const uint4*>(row + col), hi = *reinterpret_cast<const uint4*>(row + col + 8);
    const uint32_t wds[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = __uint_as_float(wds[i] << 16);
      v[2 * i + 1] = __uint_as_float(wds[i] & 0xffff0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < SSD_PER; ++i) v[i] = i < live ? to_float(row[col + i]) : 0.f;
  }
}

// A group of L lanes (a power of two, 16 states each) per (head, PP channels).  MODE 0: a request's whole portion from
// its slot's state, which is renewed.  MODE 1 (blockIdx.z = chunk): the chunk from a zero state; leaves the state it
// reaches and the product of its decays in `scratch`.  MODE 2: the chunk from the state that the carry left in
// `scratch`; writes y.  A record of `scratch` holds every thread's 16 * PP state values side by side, in the order of
// the threads (so that a chunk's state comes and goes in 16-byte pieces of whole lines), then H decay products
// (padded to a multiple of four):
// `record_floats` floats; chunk j of request b is record q_start[b] / SSD_CHUNK + b + j.
template <typename T, int PP, bool VEC, int MODE>
__global__ void __launch_bounds__(128)
ssd_scan_kernel(const T* __restrict__ xbc, int ld, const T* __restrict__ proj, int ld_proj, int dt_col,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dp,
                float* __restrict__ state, float* __restrict__ scratch, const int* __restrict__ q_start,
                const int* __restrict__ slot_ids, float* __restrict__ y, int H, int P, int N, int G, int L, int num_slots,
                size_t record_floats, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  int t0 = q_start[b], t1 = q_start[b + 1];
  size_t record = 0;
  if (MODE != 0) {
    record = (size_t)(t0 / SSD_CHUNK + b + blockIdx.z) * record_floats;
    t0 += blockIdx.z * SSD_CHUNK;
    if (t0 >= t1) return;
    t1 = min(t1, t0 + SSD_CHUNK);
  }
  const int PC = P / PP;
  const long long idx = (long long)blockIdx.y * blockDim.x + threadIdx.x;
  const int l = (int)(idx % L);
  const long long hp = idx / L;
  const bool live = hp < (long long)H * PC;  // a dead lane still takes part in the shuffles of its warp
  const int h = live ? (int)(hp / PC) : 0, p0 = live ? (int)(hp % PC) * PP : 0;
  const int slot = slot_ids[b];
  const int inner = H * P;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    if (MODE != 1 && live && l == 0)
      for (int t = t0; t < t1; ++t)
        for (int c = 0; c < PP; ++c) y[(size_t)t * inner + h * P + p0 + c] = 0.f;
    return;
  }
  const int g = h / (H / G);
  const int n0 = l * SSD_PER;
  const int states = max(0, min(SSD_PER, N - n0));
  float S[PP][SSD_PER];
  float* st = state + ((size_t)slot * H + h) * N * P + p0;                       // MODE 0: the slot, [N, P] per head
  float4* mine = reinterpret_cast<float4*>(scratch + record) + idx * (PP * SSD_PER / 4);  // else: this thread's piece
#pragma unroll
  for (int c = 0; c < PP; ++c)
#pragma unroll
    for (int i = 0; i < SSD_PER; ++i) S[c][i] = (MODE == 0 && live && i < states) ? st[(size_t)(n0 + i) * P + c] : 0.f;
  if (MODE == 2 && live) {
#pragma unroll
    for (int c = 0; c < PP; ++c)
#pragma unroll
      for (int q = 0; q < SSD_PER / 4; ++q) {
        const float4 v = mine[c * (SSD_PER / 4) + q];
        S[c][4 * q] = v.x;
        S[c][4 * q + 1] = v.y;
        S[c][4 * q + 2] = v.z;
        S[c][4 * q + 3] = v.w;
      }
  }
  constexpr bool exact = sizeof(T) == 4;
  const float rate = -expf(A_log[h]), db = dt_bias[h], dskip = Dp[h];
  const int x_col = h * P + p0, b_col = inner + g * N + n0, c_col = inner + G * N + g * N + n0;
  float log_total = 0.f;
  for (int t = t0; t < t1; ++t) {
    const T* row = xbc + (size_t)t * ld;
    const float pre = to_float(proj[(size_t)t * ld_proj + dt_col + h]) + db;
    const float step = exact ? softplus_f(pre) : fmaxf(pre, 0.f) + __logf(1.0f + __expf(-fabsf(pre)));
    const float log_a = rate * step;
    const float a = exact ? expf(log_a) : __expf(log_a);
    log_total += log_a;
    float Bv[SSD_PER], Cv[SSD_PER], x[PP];
    ssd_load16<T, VEC>(row, b_col, states, Bv);
    if (MODE != 1) ssd_load16<T, VEC>(row, c_col, states, Cv);
#pragma unroll
    for (int c = 0; c < PP; ++c) x[c] = to_float(row[x_col + c]);
#pragma unroll
    for (int c = 0; c < PP; ++c) {
      const float sx = step * x[c];
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < SSD_PER; ++i) {
        if (VEC || i < states) {
          S[c][i] = ssd_update(log_a, a, S[c][i], sx * Bv[i], exact);
          if (MODE != 1) part = fmaf(S[c][i], Cv[i], part);
        }
      }
      if (MODE != 1) {
        for (int o = L >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (live && l == 0) y[(size_t)t * inner + x_col + c] = fmaf(dskip, x[c], part);
      }
    }
  }
  if (MODE == 2 || !live) return;
  if (MODE == 1) {
#pragma unroll
    for (int c = 0; c < PP; ++c)
#pragma unroll
      for (int q = 0; q < SSD_PER / 4; ++q)
        mine[c * (SSD_PER / 4) + q] = make_float4(S[c][4 * q], S[c][4 * q + 1], S[c][4 * q + 2], S[c][4 * q + 3]);
    if (l == 0 && p0 == 0) scratch[record + record_floats - ((H + 3) & ~3) + h] = __expf(log_total);
    return;
  }
#pragma unroll
  for (int c = 0; c < PP; ++c)
#pragma unroll
    for (int i = 0; i < SSD_PER; ++i)
      if (i < states) st[(size_t)(n0 + i) * P + c] = S[c][i];
}

// One thread per state value of a request, in the order of the records (thread of the scan, channel, state): chunk
// after chunk, the record's "state reached from zero" is replaced by the state the chunk starts from,
// S_in(j + 1) = product_j S_in(j) + reached_j; the last one goes to the slot.
__global__ void ssd_carry_kernel(float* __restrict__ scratch, float* __restrict__ state, const int* __restrict__ q_start,
                                 const int* __restrict__ slot_ids, int H, int N, int P, int PP, int L, int num_slots,
                                 size_t record_floats) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const size_t e = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = slot_ids[b];
  const size_t decays_at = record_floats - ((H + 3) & ~3);
  if (e >= decays_at || slot < 0 || slot >= num_slots) return;
  const int PC = P / PP;
  const size_t thread = e / (PP * SSD_PER);
  const int within = (int)(e % (PP * SSD_PER)), c = within / SSD_PER, i = within % SSD_PER;
  const int l = (int)(thread % L);
  const size_t hp = thread / L;
  const int h = (int)(hp / PC), n = l * SSD_PER + i, p = (int)(hp % PC) * PP + c;
  if (n >= N) return;  // a lane's places beyond the last state
  const int t0 = q_start[b], chunks = (q_start[b + 1] - t0 + SSD_CHUNK - 1) / SSD_CHUNK;
  float* home = state + (((size_t)slot * H + h) * N + n) * P + p;
  float S = *home;
  float* rec = scratch + (size_t)(t0 / SSD_CHUNK + b) * record_floats;
  for (int j0 = 0; j0 < chunks; j0 += 8, rec += 8 * record_floats) {  // eight chunks' loads in flight at a time
    float reached[8], decay[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (j0 + k < chunks) {
        reached[k] = rec[(size_t)k * record_floats + e];
        decay[k] = rec[(size_t)k * record_floats + decays_at + h];
      }
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (j0 + k < chunks) {
        rec[(size_t)k * record_floats + e] = S;
        S = fmaf(decay[k], S, reached[k]);
      }
  }
  *home = S;
}

// One block per (token, part).  y: float32 [T, I]; z: [T, ld_z] at column z_col; out: [T, I].
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, int ld_z, int z_col,
                                        const float* __restrict__ weight, T* __restrict__ out, int I, int parts,
                                        float eps) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, part = blockIdx.y;
  const int width = I / parts, c0 = part * width;
  const float* yr = y + (size_t)t * I + c0;
  const T* zr = z + (size_t)t * ld_z + z_col + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = yr[i] * silu_f(to_float(zr[i]));
    ss = fmaf(v, v, ss);
  }
  const float rstd = rsqrtf(block_sum(ss, red) / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = yr[i] * silu_f(to_float(zr[i]));
    out[(size_t)t * I + c0 + i] = from_float<T>(v * rstd * weight[c0 + i]);
  }
}

}  // namespace q3

#define Q3_BY_DTYPE(dtype, CALL)                 \
  if ((dtype) == Q3_F32) { using E = float; CALL; }  \
  else if ((dtype) == Q3_BF16) { using E = __nv_bfloat16; CALL; } \
  else return Q3_ERR_DTYPE;

namespace q3 {

template <typename T, int PP, bool VEC>
static int ssd_launch(const void* xbc, int ld, const void* proj, int ld_proj, int dt_col, const float* dt_bias,
                      const float* A_log, const float* Dp, float* state, float* scratch, const int* q_start,
                      const int* slot_ids, float* y, int B, int max_q_len, int H, int P, int N, int G, int num_slots,
                      int* status, cudaStream_t stream) {
  int L = 1;
  while (L * SSD_PER < N) L <<= 1;
  const long long threads = (long long)H * (P / PP) * L;
  const long long blocks = (threads + 127) / 128;
  if (blocks > 65535) return Q3_ERR_SIZE;
  const T* x = (const T*)xbc;
  const T* pr = (const T*)proj;
  if (!scratch) {
    launch(ssd_scan_kernel<T, PP, VEC, 0>, dim3(B, (unsigned)blocks), dim3(128), 0, stream, x, ld, pr, ld_proj, dt_col,
           dt_bias, A_log, Dp, state, scratch, q_start, slot_ids, y, H, P, N, G, L, num_slots, (size_t)0, status);
    return launch_status();
  }
  const int chunks = (max_q_len + SSD_CHUNK - 1) / SSD_CHUNK;
  if (chunks > 65535) return Q3_ERR_SIZE;
  const size_t all = (size_t)threads * PP * SSD_PER, record_floats = all + ((H + 3) & ~3);
  if ((all + 255) / 256 > 65535 || record_floats % 4) return Q3_ERR_SIZE;
  launch(ssd_scan_kernel<T, PP, VEC, 1>, dim3(B, (unsigned)blocks, chunks), dim3(128), 0, stream, x, ld, pr, ld_proj,
         dt_col, dt_bias, A_log, Dp, state, scratch, q_start, slot_ids, y, H, P, N, G, L, num_slots, record_floats, status);
  launch(ssd_carry_kernel, dim3(B, (unsigned)((all + 255) / 256)), dim3(256), 0, stream, scratch, state, q_start, slot_ids,
         H, N, P, PP, L, num_slots, record_floats);
  launch(ssd_scan_kernel<T, PP, VEC, 2>, dim3(B, (unsigned)blocks, chunks), dim3(128), 0, stream, x, ld, pr, ld_proj,
         dt_col, dt_bias, A_log, Dp, state, scratch, q_start, slot_ids, y, H, P, N, G, L, num_slots, record_floats, status);
  return launch_status();
}

}  // namespace q3

extern "C" int q3_ssd_chunk() { return q3::SSD_CHUNK; }

// Floats of one record of the chunked form's scratch: 16 places per lane for every (head, channel), rounded up so that
// a record starts on a 16-byte boundary, then the heads' decay products.
extern "C" long long q3_ssd_record_floats(int H, int P, int N) {
  int L = 1;
  while (L * q3::SSD_PER < N) L <<= 1;
  return (long long)H * P * L * q3::SSD_PER + ((H + 3) & ~3);
}

// xbc: [T, ld] in `dtype`; proj: [T, ld_proj] in `dtype` with dt at dt_col; state: float32 [num_slots, H, N, P];
// y: float32 [T, H * P].  With `scratch` (float32, (T / chunk + B + 1) records of q3_ssd_record_floats; bfloat16 only)
// the portions run in chunks of q3_ssd_chunk() tokens side by side: three launches.
extern "C" int q3_ssd_scan(const void* xbc, int ld, const void* proj, int ld_proj, int dt_col, const float* dt_bias,
                           const float* A_log, const float* Dp, float* state, float* scratch, const int* q_start,
                           const int* slot_ids, float* y, int dtype, int T, int B, int max_q_len, int H, int P, int N,
                           int G, int num_slots, int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return 0;
  if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G || N > 32 * q3::SSD_PER) return Q3_ERR_SIZE;
  if (dtype == Q3_F32) {
    if (scratch) return Q3_ERR_DTYPE;  // the float32 run walks a portion in one piece, whatever its cut
    if (P % 4 == 0)
      return q3::ssd_launch<float, 4, false>(xbc, ld, proj, ld_proj, dt_col, dt_bias, A_log, Dp, state, nullptr, q_start,
                                             slot_ids, y, B, max_q_len, H, P, N, G, num_slots, status, stream);
    return q3::ssd_launch<float, 1, false>(xbc, ld, proj, ld_proj, dt_col, dt_bias, A_log, Dp, state, nullptr, q_start,
                                           slot_ids, y, B, max_q_len, H, P, N, G, num_slots, status, stream);
  }
  if (dtype != Q3_BF16) return Q3_ERR_DTYPE;
  using bf16 = __nv_bfloat16;
  const bool vec = N % 16 == 0 && (H * P) % 8 == 0 && ld % 8 == 0 && (uintptr_t)xbc % 16 == 0;
#define Q3_SSD(PP, VEC)                                                                                                  \
  return q3::ssd_launch<bf16, PP, VEC>(xbc, ld, proj, ld_proj, dt_col, dt_bias, A_log, Dp, state, scratch, q_start,      \
                                       slot_ids, y, B, max_q_len, H, P, N, G, num_slots, status, stream);
  if (P % 4 == 0) {
    if (vec) { Q3_SSD(4, true) }
    Q3_SSD(4, false)
  }
  if (vec) { Q3_SSD(1, true) }
  Q3_SSD(1, false)
#undef Q3_SSD
}

extern "C" int q3_gated_group_norm(const float* y, const void* z, int ld_z, int z_col, const float* weight, void* out,
                                   int dtype, int T, int I, int parts, float eps, cudaStream_t stream) {
  if (T <= 0 || I <= 0) return 0;
  if (parts <= 0 || I % parts || parts > 65535) return Q3_ERR_SIZE;
  int threads = ((I / parts + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  Q3_BY_DTYPE(dtype, q3::launch(q3::gated_group_norm_kernel<E>, dim3(T, parts), dim3(threads), 0, stream, y, (const E*)z,
                                ld_z, z_col, weight, (E*)out, I, parts, eps))
  return q3::launch_status();
}
