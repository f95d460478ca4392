// The state-space recurrence with one scalar decay per head (Mamba-2's), and the gated norm that follows it.
//
//   step = softplus(dt + dt_bias_h);  a = exp(-exp(A_log_h) * step)
//   S_h <- a S_h + step * B_g x_h^T        S_h: [N, P] float32, g = h / (heads / groups)
//   y_h = S_h^T C_g + D_h x_h
//
// x, B and C come from one buffer `xbc` [T, ld] (x: heads * P columns at 0, then groups * N of B, then of C), dt
// from column dt_col of `proj`.  Step sizes, decays and the state are float32 in every run.
//
// ssd_scan: a group of L lanes (a power of two, 16 states each) per (head, channel) walks a request's portion
// token by token; the lanes' parts of y meet in a butterfly of shuffles whose order is the same for every cut of
// a prompt, so the float32 run's bits do not depend on the cut.
// gated_group_norm: y * silu(z), divided by the root mean square of its part (the row is cut into equal parts),
// times a weight.
#include "common.cuh"

namespace q3 {

constexpr int SSD_PER = 16;  // states per lane

// a S + b with a = exp(log_a): see the note on slowly decaying states in seq_state.cu (the float32 run takes the
// form whose error is relative to 1 - a).
__device__ __forceinline__ float ssd_update(float log_a, float a, float S, float b, bool exact) {
  if (exact && log_a > -0.6931472f) return S + fmaf(expm1f(log_a), S, b);
  return fmaf(a, S, b);
}

template <typename T>
__global__ void __launch_bounds__(128)
ssd_scan_kernel(const T* __restrict__ xbc, int ld, const T* __restrict__ proj, int ld_proj, int dt_col,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dp,
                float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ slot_ids,
                float* __restrict__ y, int H, int P, int N, int G, int L, int num_slots, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const long long idx = (long long)blockIdx.y * blockDim.x + threadIdx.x;
  const int l = (int)(idx % L);
  const long long hp = idx / L;
  const bool live = hp < (long long)H * P;  // a dead lane still takes part in the shuffles of its warp
  const int h = live ? (int)(hp / P) : 0, p = live ? (int)(hp % P) : 0;
  const int slot = slot_ids[b];
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int inner = H * P;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    if (live && l == 0)
      for (int t = t0; t < t1; ++t) y[(size_t)t * inner + hp] = 0.f;
    return;
  }
  const int g = h / (H / G);
  const int n0 = l * SSD_PER;
  float S[SSD_PER];
  float* st = state + (((size_t)slot * H + h) * N) * P + p;
#pragma unroll
  for (int i = 0; i < SSD_PER; ++i) S[i] = (live && n0 + i < N) ? st[(size_t)(n0 + i) * P] : 0.f;
  const float rate = -expf(A_log[h]), db = dt_bias[h], dskip = Dp[h];
  const int b_col = inner + g * N + n0, c_col = inner + G * N + g * N + n0;
  constexpr bool exact = sizeof(T) == 4;
  for (int t = t0; t < t1; ++t) {
    const T* row = xbc + (size_t)t * ld;
    const float step = softplus_f(to_float(proj[(size_t)t * ld_proj + dt_col + h]) + db);
    const float log_a = rate * step;
    const float a = expf(log_a);
    const float x = to_float(row[hp < inner ? hp : 0]);
    const float sx = step * x;
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < SSD_PER; ++i) {
      if (n0 + i < N) {
        S[i] = ssd_update(log_a, a, S[i], sx * to_float(row[b_col + i]), exact);
        part = fmaf(S[i], to_float(row[c_col + i]), part);
      }
    }
    for (int o = L >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (live && l == 0) y[(size_t)t * inner + hp] = fmaf(dskip, x, part);
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < SSD_PER; ++i)
      if (n0 + i < N) st[(size_t)(n0 + i) * P] = S[i];
  }
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

// xbc: [T, ld] in `dtype`; proj: [T, ld_proj] in `dtype` with dt at dt_col; state: float32 [num_slots, H, N, P];
// y: float32 [T, H * P].
extern "C" int q3_ssd_scan(const void* xbc, int ld, const void* proj, int ld_proj, int dt_col, const float* dt_bias,
                           const float* A_log, const float* Dp, float* state, const int* q_start, const int* slot_ids,
                           float* y, int dtype, int T, int B, int H, int P, int N, int G, int num_slots, int* status,
                           cudaStream_t stream) {
  if (T <= 0 || B <= 0) return 0;
  if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G || N > 32 * q3::SSD_PER) return Q3_ERR_SIZE;
  int L = 1;
  while (L * q3::SSD_PER < N) L <<= 1;
  const long long threads = (long long)H * P * L;
  const long long blocks = (threads + 127) / 128;
  if (blocks > 65535) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::ssd_scan_kernel<E>, dim3(B, (unsigned)blocks), dim3(128), 0, stream, (const E*)xbc, ld,
                                (const E*)proj, ld_proj, dt_col, dt_bias, A_log, Dp, state, q_start, slot_ids, y, H, P, N,
                                G, L, num_slots, status))
  return q3::launch_status();
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
