// Attention whose weights are not normalised over the keys: every visible key n gets the weight
//   p_n = sigmoid((q . k_n) * scale + bias[h]),     o = gate[t, h] * sum_n p_n v_n,
// causal (a query at position p sees n <= p), grouped heads (q head h reads kv head h / (Hq / Hkv)), over the
// same paged cache as the softmax kernels.  Without a denominator the keys' contributions simply add, so a
// range of keys can be summed anywhere and the partial sums added.
//
// qk_gate_post prepares a step's projection [T, (Hq + Hkv) D + Hq]: per-head RMSNorm of q and k with a shared
// weight per kind, q times a temperature that grows with the position,
//   tau(p) = 1 + coef * ln(floor((p + 1) / every) + 1),
// the normed key into plane k of the pages and the key as projected (before the norm) into plane v: this
// design's values are its keys; and one sigmoid gate per (token, head) in float32.
//
// attn_sigmoid_kernel is the plain kernel: one warp per (query token, head), keys one by one in ascending
// position, everything float32.  It serves the float32 path, every shape, and the tests as the oracle of the
// tensor-core kernels.
#include "common.cuh"

namespace q3 {

constexpr int AS_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(AS_WARPS * 32)
qk_gate_post_kernel(const T* __restrict__ proj, int ld, int Hq, int Hkv, int D, const float* __restrict__ q_weight,
                    const float* __restrict__ k_weight, float eps, float temp_coef, int temp_every,
                    const int* __restrict__ positions, const int* __restrict__ tok_seq,
                    const int* __restrict__ block_table, int table_stride, int page_size, int num_pages,
                    T* __restrict__ k_pages, T* __restrict__ v_pages, T* __restrict__ q_out, float* __restrict__ gate_out,
                    int write_kv, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int unit = blockIdx.y * AS_WARPS + warp;
  const T* row = proj + (size_t)t * ld;
  const int pos = positions[t];
  if (unit < Hq + Hkv) {
    const T* src = row + (size_t)unit * D;
    float ss = 0.f;
    for (int e = lane; e < D; e += 32) { const float v = to_float(src[e]); ss += v * v; }
    ss = warp_sum(ss);
    const float rs = 1.0f / sqrtf(ss / (float)D + eps);
    if (unit < Hq) {
      float tau = 1.f;
      if (temp_every > 0 && pos >= 0) tau = 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
      T* dst = q_out + ((size_t)t * Hq + unit) * D;
      for (int e = lane; e < D; e += 32) dst[e] = from_float<T>(to_float(src[e]) * rs * q_weight[e] * tau);
    } else if (write_kv) {
      const int hk = unit - Hq;
      const int b = tok_seq[t];
      if (pos < 0 || b < 0) {
        if (lane == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
        return;
      }
      const int page = table_page(block_table + (size_t)b * table_stride, pos / page_size, table_stride, status);
      if (page < 0 || page >= num_pages) {
        if (lane == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
        return;
      }
      const size_t at = (((size_t)page * Hkv + hk) * page_size + (pos % page_size)) * D;
      for (int e = lane; e < D; e += 32) {
        const float v = to_float(src[e]);
        k_pages[at + e] = from_float<T>(v * rs * k_weight[e]);
        v_pages[at + e] = src[e];
      }
    }
  } else if (unit == Hq + Hkv && gate_out) {
    const T* g = row + (size_t)(Hq + Hkv) * D;
    for (int h = lane; h < Hq; h += 32) gate_out[(size_t)t * Hq + h] = sigmoid_f(to_float(g[h]));
  }
}

template <typename T, int NJ>
__global__ void __launch_bounds__(AS_WARPS * 32)
attn_sigmoid_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                    T* __restrict__ out, const float* __restrict__ head_bias, const float* __restrict__ gate,
                    const int* __restrict__ q_start, const int* __restrict__ kv_len, const int* __restrict__ tok_seq,
                    const int* __restrict__ block_table, int table_stride, int page_size, int num_pages, int Hq,
                    int Hkv, int D, float scale, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * AS_WARPS + warp;
  if (head >= Hq) return;
  const int b = tok_seq[t];
  const int q_len = q_start[b + 1] - q_start[b];
  const int pos = kv_len[b] - q_len + (t - q_start[b]);
  const int hk = head / (Hq / Hkv);
  T* o = out + ((size_t)t * Hq + head) * D;
  if (pos < 0) {
    if (lane == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    for (int e = lane; e < D; e += 32) o[e] = from_float<T>(0.f);
    return;
  }
  float qv[NJ], acc[NJ], comp[NJ];
  const T* qp = q + ((size_t)t * Hq + head) * D;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int e = lane + 32 * j;
    qv[j] = e < D ? to_float(qp[e]) : 0.f;
    acc[j] = comp[j] = 0.f;
  }
  const float hb = head_bias ? head_bias[head] : 0.f;
  const int* table = block_table + (size_t)b * table_stride;
  for (int n = 0; n <= pos; ++n) {
    const int page = table_page(table, n / page_size, table_stride, status);
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
      continue;
    }
    const size_t row = (((size_t)page * Hkv + hk) * page_size + (n % page_size)) * D;
    const T* kp = k_pages + row;
    const T* vp = v_pages + row;
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int e = lane + 32 * j;
      if (e < D) dot = fmaf(qv[j], to_float(kp[e]), dot);
    }
    dot = warp_sum(dot);
    const float p = sigmoid_f(fmaf(dot, scale, hb));
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int e = lane + 32 * j;
      if (e >= D) continue;
      if (sizeof(T) == 4) {
        // float32 run: compensated summation, so that a sum over thousands of keys stays at float32's own rounding
        const float y = fmaf(p, to_float(vp[e]), -comp[j]);
        const float tot = acc[j] + y;
        comp[j] = (tot - acc[j]) - y;
        acc[j] = tot;
      } else {
        acc[j] = fmaf(p, to_float(vp[e]), acc[j]);
      }
    }
  }
  const float g = gate ? gate[(size_t)t * Hq + head] : 1.f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int e = lane + 32 * j;
    if (e < D) o[e] = from_float<T>(acc[j] * g);
  }
}

template <typename T>
static int attn_sigmoid_launch(const void* q, const void* k_pages, const void* v_pages, void* out, const float* head_bias,
                               const float* gate, const int* q_start, const int* kv_len, const int* tok_seq,
                               const int* block_table, int table_stride, int page_size, int num_pages, int T_total, int Hq,
                               int Hkv, int D, float scale, int* status, cudaStream_t stream) {
  dim3 grid(T_total, (Hq + AS_WARPS - 1) / AS_WARPS);
  if (grid.y > 65535) return Q3_ERR_SIZE;
#define Q3_AS_CASE(NJ)                                                                                             \
  q3::launch(attn_sigmoid_kernel<T, NJ>, dim3(grid), dim3(AS_WARPS * 32), 0, stream, (const T*)q, (const T*)k_pages, \
             (const T*)v_pages, (T*)out, head_bias, gate, q_start, kv_len, tok_seq, block_table, table_stride,     \
             page_size, num_pages, Hq, Hkv, D, scale, status)
  if (D <= 32) Q3_AS_CASE(1);
  else if (D <= 64) Q3_AS_CASE(2);
  else if (D <= 128) Q3_AS_CASE(4);
  else if (D <= 256) Q3_AS_CASE(8);
  else if (D <= 512) Q3_AS_CASE(16);
  else return Q3_ERR_SIZE;
#undef Q3_AS_CASE
  return launch_status();
}

}  // namespace q3

// proj: [T, ld] in `dtype`, columns: Hq heads of q, Hkv heads of k, then Hq gate values (if gate_out).
// q_out: [T, Hq, D]; k_pages / v_pages: [num_pages, Hkv, page_size, D]; gate_out: float32 [T, Hq] or null.
// temp_every <= 0: no temperature.
extern "C" int q3_qk_gate_post(const void* proj, int dtype, int T, int ld, int Hq, int Hkv, int D, const float* q_weight,
                               const float* k_weight, float eps, float temp_coef, int temp_every, const int* positions,
                               const int* tok_seq, const int* block_table, int table_stride, int page_size, void* k_pages,
                               void* v_pages, int num_pages, void* q_out, float* gate_out, int write_kv, int* status,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (Hq <= 0 || Hkv <= 0 || D <= 0 || page_size <= 0 || table_stride <= 0 || ld < (Hq + Hkv) * D) return Q3_ERR_SIZE;
  dim3 grid(T, (Hq + Hkv + 1 + q3::AS_WARPS - 1) / q3::AS_WARPS);
  if (grid.y > 65535) return Q3_ERR_SIZE;
  if (dtype == Q3_F32)
    q3::launch(q3::qk_gate_post_kernel<float>, grid, dim3(q3::AS_WARPS * 32), 0, stream, (const float*)proj, ld, Hq, Hkv, D,
               q_weight, k_weight, eps, temp_coef, temp_every, positions, tok_seq, block_table, table_stride, page_size,
               num_pages, (float*)k_pages, (float*)v_pages, (float*)q_out, gate_out, write_kv, status);
  else if (dtype == Q3_BF16)
    q3::launch(q3::qk_gate_post_kernel<__nv_bfloat16>, grid, dim3(q3::AS_WARPS * 32), 0, stream, (const __nv_bfloat16*)proj,
               ld, Hq, Hkv, D, q_weight, k_weight, eps, temp_coef, temp_every, positions, tok_seq, block_table, table_stride,
               page_size, num_pages, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)q_out, gate_out,
               write_kv, status);
  else
    return Q3_ERR_DTYPE;
  return q3::launch_status();
}

// The plain kernel.  q, out: [T, Hq, D]; head_bias: float32 [Hq] or null; gate: float32 [T, Hq] or null.
extern "C" int q3_attn_sigmoid(const void* q, int dtype, const void* k_pages, const void* v_pages, void* out,
                               const float* head_bias, const float* gate, const int* q_start, const int* kv_len,
                               const int* tok_seq, const int* block_table, int table_stride, int page_size, int num_pages,
                               int T_total, int Hq, int Hkv, int D, float scale, int* status, cudaStream_t stream) {
  if (T_total <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || D <= 0 || page_size <= 0 || table_stride <= 0) return Q3_ERR_SIZE;
  if (dtype == Q3_F32)
    return q3::attn_sigmoid_launch<float>(q, k_pages, v_pages, out, head_bias, gate, q_start, kv_len, tok_seq, block_table,
                                          table_stride, page_size, num_pages, T_total, Hq, Hkv, D, scale, status, stream);
  if (dtype == Q3_BF16)
    return q3::attn_sigmoid_launch<__nv_bfloat16>(q, k_pages, v_pages, out, head_bias, gate, q_start, kv_len, tok_seq,
                                                  block_table, table_stride, page_size, num_pages, T_total, Hq, Hkv, D, scale,
                                                  status, stream);
  return Q3_ERR_DTYPE;
}
