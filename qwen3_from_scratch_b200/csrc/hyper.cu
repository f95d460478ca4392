// Several residual streams per token ("hyper-connections") and what stands at the two ends of such a model:
// an embedding that is scaled and copied into every stream, and a cap on the logits.
//
// The streams of a token lie side by side: xs [T, S, W] float32.  A sub-layer q reads
//     u = sum_s read[s] xs[s]                      (then a norm and the sub-layer itself: y = f(norm(u)))
// and writes, all streams at once from the old ones,
//     xs'[t] = sum_s mix[s, t] xs[s] + write[t] y  (mix is indexed [from, to]).
// One kernel closes the write of the sub-layer before (if one is still open), reads for the next one and norms:
// the streams make one trip through the memory per sub-layer, like the single stream of add_rmsnorm.
// All of it is float32; only the normed output is in the compute dtype.
#include "common.cuh"

namespace q3 {

constexpr int HC_MAX_STREAMS = 8;

// out[t, s, :] = table[ids[t]] * scale for every stream s.
template <typename T>
__global__ void embed_scaled_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                    int W, int V, int copies, float scale, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  const bool bad = id < 0 || id >= V;
  if (bad) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_TOKEN);
    id = 0;
  }
  const T* row = table + (size_t)id * W;
  float* o = out + (size_t)t * copies * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = bad ? 0.f : to_float(row[i]) * scale;
    for (int s = 0; s < copies; ++s) o[(size_t)s * W + i] = v;
  }
}

struct HcPending {  // the write of a sub-layer whose output has not reached the streams yet
  const void* delta;  // [T, W] in the compute dtype, or null: nothing is open
  const float* mix;   // [S, S], [from, to]
  const float* write; // [S]
};

// One block per row.  ROWS: the rows are chosen by `rows`, the streams are not changed and `read` is all ones
// (the sum of the streams: the model's last norm); else every row in turn and the streams are renewed in place.
template <typename T, bool ROWS>
__global__ void hc_norm_kernel(float* __restrict__ xs, HcPending pend, const float* __restrict__ read,
                               const float* __restrict__ weight, const int* __restrict__ rows, T* __restrict__ out,
                               int T_total, int S, int W, float eps, int* status) {
  __shared__ float red[32];
  __shared__ float s_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], s_write[HC_MAX_STREAMS], s_read[HC_MAX_STREAMS];
  pdl_wait();
  pdl_launch_dependents();
  int t = blockIdx.x;
  if (ROWS) {
    t = rows[blockIdx.x];
    if (t < 0 || t >= T_total) {
      if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
      for (int i = threadIdx.x; i < W; i += blockDim.x) out[(size_t)blockIdx.x * W + i] = from_float<T>(0.f);
      return;
    }
  }
  const bool open = pend.delta != nullptr;
  if (threadIdx.x < S * S) s_mix[threadIdx.x] = open ? pend.mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    s_write[threadIdx.x] = open ? pend.write[threadIdx.x] : 0.f;
    s_read[threadIdx.x] = ROWS ? 1.f : read[threadIdx.x];
  }
  __syncthreads();
  float* x = xs + (size_t)t * S * W;
  const T* delta = open ? (const T*)pend.delta + (size_t)t * W : nullptr;
  T* o = out + (size_t)blockIdx.x * W;
  float sumsq = 0.f;
  // u is kept where the output will stand?  No: the output may be narrower than float32; u is computed twice,
  // the second time from the streams as this thread left them (or, for chosen rows, in the same way again).
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float old[HC_MAX_STREAMS], u = 0.f;
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s) old[s] = s < S ? x[(size_t)s * W + i] : 0.f;
    if (open) {
      const float y = to_float(delta[i]);
#pragma unroll
      for (int to = 0; to < HC_MAX_STREAMS; ++to) {
        if (to < S) {
          float v = s_write[to] * y;
#pragma unroll
          for (int from = 0; from < HC_MAX_STREAMS; ++from)
            if (from < S) v = fmaf(s_mix[from * S + to], old[from], v);
          if (!ROWS) x[(size_t)to * W + i] = v;
          u = fmaf(s_read[to], v, u);
        }
      }
    } else {
#pragma unroll
      for (int s = 0; s < HC_MAX_STREAMS; ++s)
        if (s < S) u = fmaf(s_read[s], old[s], u);
    }
    sumsq = fmaf(u, u, sumsq);
    if (sizeof(T) == 4) o[i] = from_float<T>(u);  // float32 output: u waits in its own place
  }
  const float rstd = rsqrtf(block_sum(sumsq, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float u;
    if (sizeof(T) == 4) {
      u = to_float(o[i]);
    } else if (ROWS && open) {  // the streams were not renewed: the same sums again, in the same order
      const float y = to_float(delta[i]);
      u = 0.f;
      for (int to = 0; to < S; ++to) {
        float v = s_write[to] * y;
        for (int from = 0; from < S; ++from) v = fmaf(s_mix[from * S + to], x[(size_t)from * W + i], v);
        u = fmaf(s_read[to], v, u);
      }
    } else {
      u = 0.f;
      for (int s = 0; s < S; ++s) u = fmaf(s_read[s], x[(size_t)s * W + i], u);
    }
    o[i] = from_float<T>(u * rstd * weight[i]);
  }
}

// The same with four features per access and the row's u kept in registers: W a multiple of 4, at most
// 4 * VPT * blockDim.x; every pointer 16-byte aligned (the output 8-byte for bfloat16).
template <typename T>
__device__ __forceinline__ float4 hc_load4(const T* p);
template <>
__device__ __forceinline__ float4 hc_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 hc_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                     __uint_as_float(v.y & 0xffff0000u));
}
__device__ __forceinline__ void hc_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void hc_store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

template <typename T, bool ROWS, int VPT>
__global__ void hc_norm_vec_kernel(float* __restrict__ xs, HcPending pend, const float* __restrict__ read,
                                   const float* __restrict__ weight, const int* __restrict__ rows, T* __restrict__ out,
                                   int T_total, int S, int W, float eps, int* status) {
  __shared__ float red[32];
  __shared__ float s_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], s_write[HC_MAX_STREAMS], s_read[HC_MAX_STREAMS];
  pdl_wait();
  pdl_launch_dependents();
  int t = blockIdx.x;
  const int W4 = W >> 2;
  T* o = out + (size_t)blockIdx.x * W;
  if (ROWS) {
    t = rows[blockIdx.x];
    if (t < 0 || t >= T_total) {
      if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
      for (int f = threadIdx.x; f < W4; f += blockDim.x) hc_store4(o + 4 * f, make_float4(0.f, 0.f, 0.f, 0.f));
      return;
    }
  }
  const bool open = pend.delta != nullptr;
  if (threadIdx.x < S * S) s_mix[threadIdx.x] = open ? pend.mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    s_write[threadIdx.x] = open ? pend.write[threadIdx.x] : 0.f;
    s_read[threadIdx.x] = ROWS ? 1.f : read[threadIdx.x];
  }
  __syncthreads();
  float* x = xs + (size_t)t * S * W;
  const T* delta = open ? (const T*)pend.delta + (size_t)t * W : nullptr;
  float4 u[VPT];
  float sumsq = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int f = threadIdx.x + k * blockDim.x;
    u[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (f >= W4) continue;
    float4 old[HC_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s)
      if (s < S) old[s] = *reinterpret_cast<const float4*>(x + (size_t)s * W + 4 * f);
    if (open) {
      const float4 y = hc_load4<T>(delta + 4 * f);
#pragma unroll
      for (int to = 0; to < HC_MAX_STREAMS; ++to) {
        if (to < S) {
          const float wr = s_write[to];
          float4 v = make_float4(wr * y.x, wr * y.y, wr * y.z, wr * y.w);
#pragma unroll
          for (int from = 0; from < HC_MAX_STREAMS; ++from)
            if (from < S) {
              const float mx = s_mix[from * S + to];
              v.x = fmaf(mx, old[from].x, v.x);
              v.y = fmaf(mx, old[from].y, v.y);
              v.z = fmaf(mx, old[from].z, v.z);
              v.w = fmaf(mx, old[from].w, v.w);
            }
          if (!ROWS) *reinterpret_cast<float4*>(x + (size_t)to * W + 4 * f) = v;
          const float rd = s_read[to];
          u[k].x = fmaf(rd, v.x, u[k].x);
          u[k].y = fmaf(rd, v.y, u[k].y);
          u[k].z = fmaf(rd, v.z, u[k].z);
          u[k].w = fmaf(rd, v.w, u[k].w);
        }
      }
    } else {
#pragma unroll
      for (int s = 0; s < HC_MAX_STREAMS; ++s)
        if (s < S) {
          const float rd = s_read[s];
          u[k].x = fmaf(rd, old[s].x, u[k].x);
          u[k].y = fmaf(rd, old[s].y, u[k].y);
          u[k].z = fmaf(rd, old[s].z, u[k].z);
          u[k].w = fmaf(rd, old[s].w, u[k].w);
        }
    }
    sumsq = fmaf(u[k].x, u[k].x, fmaf(u[k].y, u[k].y, fmaf(u[k].z, u[k].z, fmaf(u[k].w, u[k].w, sumsq))));
  }
  const float rstd = rsqrtf(block_sum(sumsq, red) / (float)W + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int f = threadIdx.x + k * blockDim.x;
    if (f >= W4) continue;
    const float4 wv = *reinterpret_cast<const float4*>(weight + 4 * f);
    hc_store4(o + 4 * f, make_float4(u[k].x * rstd * wv.x, u[k].y * rstd * wv.y, u[k].z * rstd * wv.z, u[k].w * rstd * wv.w));
  }
}

template <typename T, bool ROWS>
static bool hc_launch_vec(float* xs, HcPending pend, const float* read, const float* weight, const int* rows, void* out,
                          int blocks, int T_total, int S, int W, float eps, int* status, cudaStream_t stream) {
  if (W % 4 || (uintptr_t)xs % 16 || (uintptr_t)weight % 16 || (uintptr_t)out % 16 || (pend.delta && (uintptr_t)pend.delta % 16))
    return false;
  const int W4 = W / 4;
  if (W4 > 256 * 4) return false;
  int threads = W4 <= 256 ? ((W4 + 31) / 32) * 32 : 256;
  if (threads < 64) threads = 64;
  const int vpt = (W4 + threads - 1) / threads;
  if (vpt == 1)
    launch(hc_norm_vec_kernel<T, ROWS, 1>, dim3(blocks), dim3(threads), 0, stream, xs, pend, read, weight, rows, (T*)out,
           T_total, S, W, eps, status);
  else if (vpt == 2)
    launch(hc_norm_vec_kernel<T, ROWS, 2>, dim3(blocks), dim3(threads), 0, stream, xs, pend, read, weight, rows, (T*)out,
           T_total, S, W, eps, status);
  else
    launch(hc_norm_vec_kernel<T, ROWS, 4>, dim3(blocks), dim3(threads), 0, stream, xs, pend, read, weight, rows, (T*)out,
           T_total, S, W, eps, status);
  return true;
}

// logits <- cap * tanh(logits / cap), in place, float32.
__global__ void softcap_kernel(float* __restrict__ logits, size_t total, float cap) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) logits[i] = cap * tanhf(logits[i] / cap);
}

}  // namespace q3

#define Q3_BY_DTYPE(dtype, CALL)                 \
  if ((dtype) == Q3_F32) { using E = float; CALL; }  \
  else if ((dtype) == Q3_BF16) { using E = __nv_bfloat16; CALL; } \
  else return Q3_ERR_DTYPE;

// out: float32 [T, copies, W]; table: [V, W] in `dtype`.
extern "C" int q3_embed_scaled(const void* table, int dtype, const int* ids, float* out, int T, int W, int V, int copies,
                               float scale, int* status, cudaStream_t stream) {
  if (T <= 0 || W <= 0) return 0;
  if (copies <= 0) return Q3_ERR_SIZE;
  int threads = ((W + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  Q3_BY_DTYPE(dtype, q3::launch(q3::embed_scaled_kernel<E>, dim3(T), dim3(threads), 0, stream, (const E*)table, ids, out, W,
                                V, copies, scale, status))
  q3::note_stream_written();
  return q3::launch_status();
}

// xs: float32 [T, S, W], renewed in place when a write is open (delta: [T, W] in `dtype`, mix [S, S], write [S]);
// out: [T, W] in `dtype` = rmsnorm(sum_s read[s] xs[s]) * weight.
extern "C" int q3_hc_norm(float* xs, const void* delta, const float* mix, const float* write, const float* read,
                          const float* weight, void* out, int dtype, int T, int S, int W, float eps, int* status,
                          cudaStream_t stream) {
  if (T <= 0 || W <= 0) return 0;
  if (S <= 0 || S > q3::HC_MAX_STREAMS) return Q3_ERR_SIZE;
  int threads = ((W + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  if (threads < 64) threads = 64;  // the first S * S threads fetch the mixing matrix
  q3::HcPending pend{delta, mix, write};
  Q3_BY_DTYPE(dtype, {
    if (!q3::hc_launch_vec<E, false>(xs, pend, read, weight, nullptr, out, T, T, S, W, eps, status, stream))
      q3::launch(q3::hc_norm_kernel<E, false>, dim3(T), dim3(threads), 0, stream, xs, pend, read, weight,
                 (const int*)nullptr, (E*)out, T, S, W, eps, status);
  })
  if (delta) q3::note_stream_written();
  return q3::launch_status();
}

// out: [R, W] in `dtype` = rmsnorm(sum of the streams of row rows[r], with the open write applied) * weight; the
// streams stay as they are.
extern "C" int q3_hc_sum_norm_rows(const float* xs, const void* delta, const float* mix, const float* write,
                                   const float* weight, const int* rows, void* out, int dtype, int T, int R, int S, int W,
                                   float eps, int* status, cudaStream_t stream) {
  if (R <= 0 || W <= 0) return 0;
  if (S <= 0 || S > q3::HC_MAX_STREAMS) return Q3_ERR_SIZE;
  int threads = ((W + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  if (threads < 64) threads = 64;
  q3::HcPending pend{delta, mix, write};
  Q3_BY_DTYPE(dtype, {
    if (!q3::hc_launch_vec<E, true>((float*)xs, pend, nullptr, weight, rows, out, R, T, S, W, eps, status, stream))
      q3::launch(q3::hc_norm_kernel<E, true>, dim3(R), dim3(threads), 0, stream, (float*)xs, pend, (const float*)nullptr,
                 weight, rows, (E*)out, T, S, W, eps, status);
  })
  return q3::launch_status();
}

extern "C" int q3_softcap(float* logits, long long total, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) return Q3_ERR_SIZE;
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffll) return Q3_ERR_SIZE;
  q3::launch(q3::softcap_kernel, dim3((unsigned)blocks), dim3(threads), 0, stream, logits, (size_t)total, cap);
  return q3::launch_status();
}
