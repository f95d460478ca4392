// The state-space recurrence of ssd.cu in its matrix form, on the tensor cores (bfloat16 run, prompt portions).
//
// Within a chunk of SM_Q tokens of one head, with a_t = log of the decay, cum_t = a_1 + .. + a_t (inclusive) and
// step_t the step size, the recurrence S_t = e^{a_t} S_{t-1} + step_t B_t x_t^T, y_t = S_t^T C_t + D x_t unrolls to
//
//   y_t      = sum_{s <= t} (C_t . B_s) e^{cum_t - cum_s} step_s x_s  +  e^{cum_t} C_t^T S_in  +  D x_t
//   S_out    = e^{cum_last} S_in + sum_s e^{cum_last - cum_s} step_s B_s x_s^T
//
// so a chunk is three matrix products: G = C B^T (then M = G masked and weighted), M X, and C S_in; and its
// contribution to the state is one more, B^T (w . X).  Launches: ssd_chunk_state (every chunk's state reached from
// zero and the product of its decays), the carry (chunk after chunk, S_in(j + 1) = product_j S_in(j) + reached_j; it
// leaves S_in(j) in the record), ssd_chunk_output (y of every chunk).
//
// What enters a product must be bfloat16.  x, B and C are (they are the convolution's output).  Everything that
// carries a decay, a step size or the state is float32 and is split into two bfloat16 halves, v = hi + lo with
// lo = bf16(v - hi), and multiplied in two products (the other operand is exact), which keeps about 16 bits of each
// instead of 8; e^{cum_t} multiplies the finished rows of C S_in in float32, so C itself stays as it is.
// Accumulation is float32.  The float32 run does not come here: it walks token by token (ssd.cu).
#include "attn_mma.cuh"

namespace q3 {

constexpr int SM_Q = 64;  // tokens per chunk (the same as ssd.cu's, whose carry's record index this shares)

__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(v);
  lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

// What both kernels do first: the chunk's rows of x (this head's P channels), B and C (its group's N values) into
// shared memory as [SM_Q][P + 8] and [SM_Q][N + 8], zero beyond the chunk's end; step sizes and the inclusive sums of
// the log-decays (a row beyond the end has step 0 and decay 1: it changes nothing).
template <int P, int N, bool WANT_C>
__device__ __forceinline__ void load_chunk(const __nv_bfloat16* __restrict__ xbc, int ld, const __nv_bfloat16* __restrict__ proj,
                                           int ld_proj, int dt_col, int h, int g, int G, int inner, float rate, float db,
                                           int t0, int len, __nv_bfloat16* xs, __nv_bfloat16* bs, __nv_bfloat16* cs,
                                           float* step_s, float* cum_s) {
  constexpr int PX = P + 8, PN = N + 8;
  for (int i = threadIdx.x; i < SM_Q * (P / 8); i += blockDim.x) {
    const int t = i / (P / 8), c = i % (P / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < len) v = *reinterpret_cast<const uint4*>(xbc + (size_t)(t0 + t) * ld + h * P + c * 8);
    *reinterpret_cast<uint4*>(xs + t * PX + c * 8) = v;
  }
  for (int i = threadIdx.x; i < SM_Q * (N / 8); i += blockDim.x) {
    const int t = i / (N / 8), c = i % (N / 8);
    uint4 vb = make_uint4(0, 0, 0, 0), vc = make_uint4(0, 0, 0, 0);
    if (t < len) {
      const __nv_bfloat16* row = xbc + (size_t)(t0 + t) * ld + inner + g * N + c * 8;
      vb = *reinterpret_cast<const uint4*>(row);
      if (WANT_C) vc = *reinterpret_cast<const uint4*>(row + (size_t)G * N);
    }
    *reinterpret_cast<uint4*>(bs + t * PN + c * 8) = vb;
    if (WANT_C) *reinterpret_cast<uint4*>(cs + t * PN + c * 8) = vc;
  }
  if (threadIdx.x < SM_Q) {
    const int t = threadIdx.x;
    float step = 0.f;
    if (t < len) {
      const float pre = __bfloat162float(proj[(size_t)(t0 + t) * ld_proj + dt_col + h]) + db;
      step = fmaxf(pre, 0.f) + __logf(1.0f + __expf(-fabsf(pre)));
    }
    step_s[t] = step;
    cum_s[t] = rate * step;  // the log-decay, summed below
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // 64 additions in the order of the tokens
    float run = 0.f;
    for (int t = 0; t < SM_Q; ++t) {
      run += cum_s[t];
      cum_s[t] = run;
    }
  }
  __syncthreads();
}

// grid (requests, chunks, heads), 128 threads.  Leaves in the chunk's record: reached[h][n][p] =
// sum_s e^{cum_last - cum_s} step_s B_s[n] x_s[p] (float32) and, after the H * N * P states, the decay product of the head.
template <int P, int N>
__global__ void __launch_bounds__(128)
ssd_chunk_state_kernel(const __nv_bfloat16* __restrict__ xbc, int ld, const __nv_bfloat16* __restrict__ proj, int ld_proj,
                       int dt_col, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                       float* __restrict__ scratch, const int* __restrict__ q_start, const int* __restrict__ slot_ids, int H,
                       int G, int num_slots, size_t record_floats) {
  constexpr int PX = P + 8, PN = N + 8;
  extern __shared__ __align__(16) unsigned char sm_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(sm_raw);  // [SM_Q][PX]
  __nv_bfloat16* bs = xs + SM_Q * PX;                            // [SM_Q][PN]
  __nv_bfloat16* xw_hi = bs + SM_Q * PN;                         // [SM_Q][PX]: w_s x_s, upper half
  __nv_bfloat16* xw_lo = xw_hi + SM_Q * PX;
  float* step_s = reinterpret_cast<float*>(xw_lo + SM_Q * PX);
  float* cum_s = step_s + SM_Q;
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.z;
  const int slot = slot_ids[b];
  const int start = q_start[b], t0 = start + blockIdx.y * SM_Q, t1 = q_start[b + 1];
  if (t0 >= t1 || slot < 0 || slot >= num_slots) return;
  const int len = min(SM_Q, t1 - t0);
  const int inner = H * P, g = h / (H / G);
  load_chunk<P, N, false>(xbc, ld, proj, ld_proj, dt_col, h, g, G, inner, -expf(A_log[h]), dt_bias[h], t0, len, xs, bs,
                          nullptr, step_s, cum_s);
  const float last = cum_s[SM_Q - 1];
  for (int i = threadIdx.x; i < SM_Q * P; i += blockDim.x) {
    const int s = i / P, p = i % P;
    const float w = __expf(last - cum_s[s]) * step_s[s];
    split_bf16(w * __bfloat162float(xs[s * PX + p]), xw_hi[s * PX + p], xw_lo[s * PX + p]);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tid4 = lane & 3;
  constexpr int MT = N / 64;  // 16-row tiles of the N state rows per warp
  float v[MT][P / 8][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < P / 8; ++i) v[m][i][0] = v[m][i][1] = v[m][i][2] = v[m][i][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < SM_Q / 16; ++ks) {  // the reduction runs over the chunk's tokens
    uint32_t af[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)  // A[n][s] = B_s[n]: the stored [s][n] tile, transposed on the way
      ldmatrix_x4_trans(af[m], bs + (ks * 16 + (lane & 7) + ((lane >> 4) << 3)) * PN + (warp * MT + m) * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
    for (int dt = 0; dt < P / 16; ++dt) {
      uint32_t hi[4], lo[4];
      const int at = (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PX + dt * 16 + (lane >> 4) * 8;
      ldmatrix_x4_trans(hi, xw_hi + at);
      ldmatrix_x4_trans(lo, xw_lo + at);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        mma_bf16(v[m][2 * dt], af[m], hi[0], hi[1]);
        mma_bf16(v[m][2 * dt + 1], af[m], hi[2], hi[3]);
        mma_bf16(v[m][2 * dt], af[m], lo[0], lo[1]);
        mma_bf16(v[m][2 * dt + 1], af[m], lo[2], lo[3]);
      }
    }
  }
  float* rec = scratch + (size_t)(start / SM_Q + b + blockIdx.y) * record_floats;
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < P / 8; ++i)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int n = (warp * MT + m) * 16 + gid + 8 * r, p = i * 8 + 2 * tid4;
        *reinterpret_cast<float2*>(rec + ((size_t)h * N + n) * P + p) = make_float2(v[m][i][2 * r], v[m][i][2 * r + 1]);
      }
  if (threadIdx.x == 0) rec[(size_t)H * N * P + h] = __expf(last);
}

// One thread per state value: the records' "reached from zero" become "the state the chunk starts from", the last
// state goes to the slot.  Records and slot both [H][N][P].
__global__ void ssd_chunk_carry_kernel(float* __restrict__ scratch, float* __restrict__ state, const int* __restrict__ q_start,
                                       const int* __restrict__ slot_ids, int H, int NP, int num_slots, size_t record_floats) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const size_t e = (size_t)blockIdx.y * blockDim.x + threadIdx.x, all = (size_t)H * NP;
  const int slot = slot_ids[b];
  if (e >= all || slot < 0 || slot >= num_slots) return;
  const int t0 = q_start[b], chunks = (q_start[b + 1] - t0 + SM_Q - 1) / SM_Q;
  const int h = (int)(e / NP);
  float S = state[(size_t)slot * all + e];
  float* rec = scratch + (size_t)(t0 / SM_Q + b) * record_floats;
  for (int j0 = 0; j0 < chunks; j0 += 8, rec += 8 * record_floats) {  // eight chunks' loads in flight at a time
    float reached[8], decay[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (j0 + k < chunks) {
        reached[k] = rec[(size_t)k * record_floats + e];
        decay[k] = rec[(size_t)k * record_floats + all + h];
      }
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (j0 + k < chunks) {
        rec[(size_t)k * record_floats + e] = S;
        S = fmaf(decay[k], S, reached[k]);
      }
  }
  state[(size_t)slot * all + e] = S;
}

// grid (requests, chunks, heads), 128 threads: warp w owns the chunk's rows 16 w .. 16 w + 15.
template <int P, int N>
__global__ void __launch_bounds__(128)
ssd_chunk_output_kernel(const __nv_bfloat16* __restrict__ xbc, int ld, const __nv_bfloat16* __restrict__ proj, int ld_proj,
                        int dt_col, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                        const float* __restrict__ Dp, const float* __restrict__ scratch, const int* __restrict__ q_start,
                        const int* __restrict__ slot_ids, float* __restrict__ y, int H, int G, int num_slots,
                        size_t record_floats) {
  constexpr int PX = P + 8, PN = N + 8;
  extern __shared__ __align__(16) unsigned char sm_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(sm_raw);  // [SM_Q][PX]
  __nv_bfloat16* bs = xs + SM_Q * PX;                            // [SM_Q][PN]
  __nv_bfloat16* cs = bs + SM_Q * PN;                            // [SM_Q][PN]
  __nv_bfloat16* s_hi = cs + SM_Q * PN;                          // [N][PX]: the state the chunk starts from
  __nv_bfloat16* s_lo = s_hi + N * PX;
  float* step_s = reinterpret_cast<float*>(s_lo + N * PX);
  float* cum_s = step_s + SM_Q;
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.z;
  const int slot = slot_ids[b];
  const int start = q_start[b], t0 = start + blockIdx.y * SM_Q, t1 = q_start[b + 1];
  if (t0 >= t1) return;
  const int len = min(SM_Q, t1 - t0);
  const int inner = H * P, g = h / (H / G);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tid4 = lane & 3;
  if (slot < 0 || slot >= num_slots) {
    for (int i = threadIdx.x; i < len * P; i += blockDim.x) y[(size_t)(t0 + i / P) * inner + h * P + i % P] = 0.f;
    return;
  }
  const float* rec = scratch + (size_t)(start / SM_Q + b + blockIdx.y) * record_floats + (size_t)h * N * P;
  for (int i = threadIdx.x; i < N * P / 4; i += blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(rec)[i];
    const int n = (4 * i) / P, p = (4 * i) % P;
    const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) split_bf16(vv[k], s_hi[n * PX + p + k], s_lo[n * PX + p + k]);
  }
  load_chunk<P, N, true>(xbc, ld, proj, ld_proj, dt_col, h, g, G, inner, -expf(A_log[h]), dt_bias[h], t0, len, xs, bs, cs,
                         step_s, cum_s);
  // this warp's rows of C as A fragments, for G = C B^T and for C S_in
  uint32_t cf[N / 16][4];
#pragma unroll
  for (int ks = 0; ks < N / 16; ++ks) ldmatrix_x4(cf[ks], cs + (warp * 16 + (lane & 15)) * PN + ks * 16 + (lane >> 4) * 8);
  // G[t][s] = C_t . B_s
  float gacc[SM_Q / 8][4];
#pragma unroll
  for (int i = 0; i < SM_Q / 8; ++i) gacc[i][0] = gacc[i][1] = gacc[i][2] = gacc[i][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < N / 16; ++ks)
#pragma unroll
    for (int np = 0; np < SM_Q / 16; ++np) {
      uint32_t kb[4];
      ldmatrix_x4(kb, bs + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * PN + ks * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(gacc[2 * np], cf[ks], kb[0], kb[1]);
      mma_bf16(gacc[2 * np + 1], cf[ks], kb[2], kb[3]);
    }
  // M[t][s] = G[t][s] e^{cum_t - cum_s} step_s for s <= t, in two halves, as A fragments
  const int tr[2] = {warp * 16 + gid, warp * 16 + gid + 8};
  const float cum_t[2] = {cum_s[tr[0]], cum_s[tr[1]]};
  uint32_t m_hi[SM_Q / 16][4], m_lo[SM_Q / 16][4];
#pragma unroll
  for (int nt = 0; nt < SM_Q / 8; ++nt) {
    __nv_bfloat16 hi[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = j >> 1, s = nt * 8 + 2 * tid4 + (j & 1);
      const float m = s <= tr[r] ? gacc[nt][j] * __expf(cum_t[r] - cum_s[s]) * step_s[s] : 0.f;
      split_bf16(m, hi[j], lo[j]);
    }
    const int kk = nt >> 1, half = (nt & 1) * 2;  // n-tile 2 kk fills registers 0, 1 of k-step kk; 2 kk + 1 fills 2, 3
    m_hi[kk][half] = pack_bf16(__bfloat162float(hi[0]), __bfloat162float(hi[1]));
    m_hi[kk][half + 1] = pack_bf16(__bfloat162float(hi[2]), __bfloat162float(hi[3]));
    m_lo[kk][half] = pack_bf16(__bfloat162float(lo[0]), __bfloat162float(lo[1]));
    m_lo[kk][half + 1] = pack_bf16(__bfloat162float(lo[2]), __bfloat162float(lo[3]));
  }
  // y = M X + e^{cum_t} (C S_in) + D x
  float acc[P / 8][4], z[P / 8][4];
#pragma unroll
  for (int i = 0; i < P / 8; ++i) {
    acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    z[i][0] = z[i][1] = z[i][2] = z[i][3] = 0.f;
  }
#pragma unroll
  for (int kk = 0; kk < SM_Q / 16; ++kk)
#pragma unroll
    for (int dt = 0; dt < P / 16; ++dt) {
      uint32_t vb[4];
      ldmatrix_x4_trans(vb, xs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PX + dt * 16 + (lane >> 4) * 8);
      mma_bf16(acc[2 * dt], m_hi[kk], vb[0], vb[1]);
      mma_bf16(acc[2 * dt + 1], m_hi[kk], vb[2], vb[3]);
      mma_bf16(acc[2 * dt], m_lo[kk], vb[0], vb[1]);
      mma_bf16(acc[2 * dt + 1], m_lo[kk], vb[2], vb[3]);
    }
#pragma unroll
  for (int ks = 0; ks < N / 16; ++ks)
#pragma unroll
    for (int dt = 0; dt < P / 16; ++dt) {
      uint32_t hi[4], lo[4];
      const int at = (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PX + dt * 16 + (lane >> 4) * 8;
      ldmatrix_x4_trans(hi, s_hi + at);
      ldmatrix_x4_trans(lo, s_lo + at);
      mma_bf16(z[2 * dt], cf[ks], hi[0], hi[1]);
      mma_bf16(z[2 * dt + 1], cf[ks], hi[2], hi[3]);
      mma_bf16(z[2 * dt], cf[ks], lo[0], lo[1]);
      mma_bf16(z[2 * dt + 1], cf[ks], lo[2], lo[3]);
    }
  const float dskip = Dp[h];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (tr[r] >= len) continue;
    const float e = __expf(cum_t[r]);
    float* dst = y + (size_t)(t0 + tr[r]) * inner + h * P;
#pragma unroll
    for (int i = 0; i < P / 8; ++i) {
      const int p = i * 8 + 2 * tid4;
      const float x0 = __bfloat162float(xs[tr[r] * PX + p]), x1 = __bfloat162float(xs[tr[r] * PX + p + 1]);
      *reinterpret_cast<float2*>(dst + p) = make_float2(acc[i][2 * r] + fmaf(e, z[i][2 * r], dskip * x0),
                                                        acc[i][2 * r + 1] + fmaf(e, z[i][2 * r + 1], dskip * x1));
    }
  }
}

template <int P, int N>
static int ssd_mma_launch(const void* xbc, int ld, const void* proj, int ld_proj, int dt_col, const float* dt_bias,
                          const float* A_log, const float* Dp, float* state, float* scratch, const int* q_start,
                          const int* slot_ids, float* y, int B, int max_q_len, int H, int G, int num_slots,
                          cudaStream_t stream) {
  using bf16 = __nv_bfloat16;
  constexpr int PX = P + 8, PN = N + 8;
  const size_t smem1 = (size_t)(3 * SM_Q * PX + SM_Q * PN) * sizeof(bf16) + 2 * SM_Q * sizeof(float);
  const size_t smem2 = (size_t)(SM_Q * PX + 2 * SM_Q * PN + 2 * N * PX) * sizeof(bf16) + 2 * SM_Q * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(ssd_chunk_state_kernel<P, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    cudaFuncSetAttribute(ssd_chunk_output_kernel<P, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    configured = true;
  }
  const int chunks = (max_q_len + SM_Q - 1) / SM_Q;
  const size_t all = (size_t)H * N * P, record_floats = all + ((H + 3) & ~3);
  if (chunks > 65535 || H > 65535 || (all + 255) / 256 > 65535) return Q3_ERR_SIZE;
  launch(ssd_chunk_state_kernel<P, N>, dim3(B, chunks, H), dim3(128), smem1, stream, (const bf16*)xbc, ld, (const bf16*)proj,
         ld_proj, dt_col, dt_bias, A_log, scratch, q_start, slot_ids, H, G, num_slots, record_floats);
  launch(ssd_chunk_carry_kernel, dim3(B, (unsigned)((all + 255) / 256)), dim3(256), 0, stream, scratch, state, q_start,
         slot_ids, H, N * P, num_slots, record_floats);
  launch(ssd_chunk_output_kernel<P, N>, dim3(B, chunks, H), dim3(128), smem2, stream, (const bf16*)xbc, ld,
         (const bf16*)proj, ld_proj, dt_col, dt_bias, A_log, Dp, (const float*)scratch, q_start, slot_ids, y, H, G,
         num_slots, record_floats);
  return launch_status();
}

}  // namespace q3

// 1 if the matrix form takes these sizes: heads of 64 channels, a state of 64 or 128.
extern "C" int q3_ssd_mma_takes(int P, int N) { return P == 64 && (N == 64 || N == 128) ? 1 : 0; }

// Floats of one record of its scratch ((T / 64 + B + 1) records): a head-major state and the heads' decay products.
extern "C" long long q3_ssd_mma_record_floats(int H, int P, int N) { return (long long)H * N * P + ((H + 3) & ~3); }

// The arguments of q3_ssd_scan (bfloat16 only; scratch is required).
extern "C" int q3_ssd_scan_mma(const void* xbc, int ld, const void* proj, int ld_proj, int dt_col, const float* dt_bias,
                               const float* A_log, const float* Dp, float* state, float* scratch, const int* q_start,
                               const int* slot_ids, float* y, int T, int B, int max_q_len, int H, int P, int N, int G,
                               int num_slots, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return 0;
  if (!q3_ssd_mma_takes(P, N) || H <= 0 || G <= 0 || H % G || !scratch) return Q3_ERR_SIZE;
  if (ld % 8 || (H * P) % 8 || (uintptr_t)xbc % 16 || (uintptr_t)scratch % 16 || (uintptr_t)y % 8) return Q3_ERR_ALIGN;
  if (N == 64)
    return q3::ssd_mma_launch<64, 64>(xbc, ld, proj, ld_proj, dt_col, dt_bias, A_log, Dp, state, scratch, q_start, slot_ids,
                                      y, B, max_q_len, H, G, num_slots, stream);
  return q3::ssd_mma_launch<64, 128>(xbc, ld, proj, ld_proj, dt_col, dt_bias, A_log, Dp, state, scratch, q_start, slot_ids,
                                     y, B, max_q_len, H, G, num_slots, stream);
}
