// Sigmoid-weighted paged causal attention on the tensor cores (bfloat16; see attn_sigmoid.cu for the formula
// and the plain kernel that is its oracle), in two forms of one kernel:
//
//   portions  grid (query tile, kv head, sequence): 128 (64 for large heads) rows of (token, head-in-group)
//             pairs, one 16-row slice per warp, all keys up to the tile's last position in tiles of 64.
//   decode    grid (key range, kv head, sequence), one token per sequence: the g heads of the group are the
//             (padded) 16 rows of every warp, and the four warps share each 64-key tile, 16 keys each.  The
//             warps' sums are added through shared memory; with several key ranges each block leaves a float32
//             partial sum and sum_gate_kernel adds them in a fixed order.
//
// Without a softmax there is no running maximum, no denominator and nothing to rescale: S = Q K^T
// (m16n8k16, float32 accumulate), p = sigmoid(S * scale + b_h) in float32 with masked keys at exactly 0,
// O += P V with P rounded to bfloat16, and the head's gate multiplies the finished row.
// Keys and values come from the pages by cp.async, two stages.
#include "attn_mma.cuh"

namespace q3 {

constexpr int SM_BN = 64;  // keys per tile

template <int KT, bool DECODE>
struct SigmoidShape {
  static constexpr int D = 16 * KT;
  static constexpr int PITCH = D + 8;
  static constexpr int TILE = SM_BN * PITCH;
  static constexpr int WARPS = DECODE ? 4 : (KT <= 8 ? 8 : 4);
  static constexpr int BM = DECODE ? 16 : 16 * WARPS;
  static constexpr int NP = DECODE ? 1 : 4;  // pairs of 8-key columns per warp and tile
  static constexpr size_t KV_BYTES = sizeof(__nv_bfloat16) * (size_t)(BM * PITCH + 4 * TILE);
  static constexpr size_t RED_BYTES = DECODE ? sizeof(float) * (size_t)(WARPS * 16 * (D + 1)) : 0;
  static constexpr size_t SMEM_BYTES = KV_BYTES > RED_BYTES ? KV_BYTES : RED_BYTES;
};

__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

template <int KT, bool DECODE>
__global__ void __launch_bounds__(SigmoidShape<KT, DECODE>::WARPS * 32)
attn_sigmoid_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ partial, const float* __restrict__ head_bias,
                        const float* __restrict__ gate, const int* __restrict__ q_start,
                        const int* __restrict__ kv_len, const int* __restrict__ block_table, int table_stride,
                        int page_size, int num_pages, int Hq, int Hkv, float scale, int num_splits, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  using S = SigmoidShape<KT, DECODE>;
  constexpr int D = S::D, PITCH = S::PITCH, TILE = S::TILE, CPR = D / 8, NP = S::NP;
  constexpr int WARPS = S::WARPS, BM = S::BM;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* kv_s = q_s + BM * PITCH;  // [stage][K | V][64][PITCH]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tid4 = lane & 3;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int g = Hq / Hkv;
  const int qs = q_start[b];
  const int q_len = DECODE ? 1 : q_start[b + 1] - qs;
  const int len = kv_len[b];
  const int total_rows = q_len * g;
  const int row0 = DECODE ? 0 : blockIdx.x * BM;
  if (row0 >= total_rows) return;
  const int past = len - q_len;  // position of this step's first token
  if (past < 0) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    return;
  }
  const int* table = block_table + (size_t)b * table_stride;
  const int last_row = min(total_rows, row0 + BM) - 1;
  const int pos_first = past + row0 / g, pos_last = past + last_row / g;
  int tile_lo = 0, tile_hi = pos_last / SM_BN;
  if (DECODE) {  // this block's share of the key tiles
    const int tiles = tile_hi + 1, per = (tiles + num_splits - 1) / num_splits;
    tile_lo = blockIdx.x * per;
    tile_hi = min(tile_hi, tile_lo + per - 1);
  }

  for (int e = threadIdx.x; e < BM * CPR; e += WARPS * 32) {
    const int rr = e / CPR, c = e % CPR;
    const int R = row0 + rr;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < total_rows)
      v = *reinterpret_cast<const uint4*>(q + ((size_t)(qs + R / g) * Hq + hk * g + R % g) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + rr * PITCH + c * 8) = v;
  }

  constexpr int LANES_PER_ROW = WARPS * 32 / SM_BN;  // threads that share a key row: 2 or 4
  auto load_tile = [&](int tile, int stage) {
    const int row = threadIdx.x / LANES_PER_ROW, part = threadIdx.x % LANES_PER_ROW;
    const int n = tile * SM_BN + row;
    const __nv_bfloat16 *ks = k_pages, *vs = v_pages;
    int bytes = 0;
    if (n <= pos_last) {
      const int page = table_page(table, n / page_size, table_stride, status);
      if (page >= 0 && page < num_pages) {
        const size_t off = (((size_t)page * Hkv + hk) * page_size + (n % page_size)) * D;
        ks = k_pages + off;
        vs = v_pages + off;
        bytes = 16;
      } else {
        atomicOr(status, Q3_STATUS_BAD_PAGE);
      }
    }
    __nv_bfloat16* kd = kv_s + (size_t)(stage * 2) * TILE + row * PITCH;
    __nv_bfloat16* vd = kd + TILE;
#pragma unroll
    for (int c = part; c < CPR; c += LANES_PER_ROW) {
      const int src = bytes ? c * 8 : 0;
      cp_async_16(kd + c * 8, ks + src, bytes);
      cp_async_16(vd + c * 8, vs + src, bytes);
    }
  };

  float o[2 * KT][4];
#pragma unroll
  for (int i = 0; i < 2 * KT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  // the two rows this thread owns in the score and output fragments
  const int warp_row = DECODE ? 0 : warp * 16;
  int row_pos[2];
  float row_bias[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int R = row0 + warp_row + gid + 8 * r;
    row_pos[r] = R < total_rows ? past + R / g : -1;  // rows past the end see no key
    row_bias[r] = (head_bias && R < total_rows) ? head_bias[hk * g + R % g] : 0.f;
  }

  if (tile_lo <= tile_hi) {
    load_tile(tile_lo, 0);
    cp_async_commit();
    __syncthreads();  // the query tile is in place
    const __nv_bfloat16* q_warp = q_s + (warp_row + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + (lane >> 4) * 8;
    const int key0 = DECODE ? warp * 16 : 0;  // this warp's first key row of a tile

    for (int tile = tile_lo; tile <= tile_hi; ++tile) {
      const int stage = (tile - tile_lo) & 1;
      if (tile + 1 <= tile_hi) load_tile(tile + 1, stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();
      const __nv_bfloat16* kt_s = kv_s + (size_t)(stage * 2) * TILE;
      const __nv_bfloat16* vt_s = kt_s + TILE;

      float s[2 * NP][4];
#pragma unroll
      for (int i = 0; i < 2 * NP; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kt = 0; kt < KT; ++kt) {
        uint32_t qf[4];
        ldmatrix_x4(qf, q_warp + kt * 16);
#pragma unroll
        for (int np = 0; np < NP; ++np) {
          uint32_t kb[4];
          ldmatrix_x4(kb, kt_s + (key0 + np * 16 + (lane & 7) + ((lane >> 4) << 3)) * PITCH + kt * 16 +
                              ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * np], qf, kb[0], kb[1]);
          mma_bf16(s[2 * np + 1], qf, kb[2], kb[3]);
        }
      }
      const int base_n = tile * SM_BN + key0;
#pragma unroll
      for (int nt = 0; nt < 2 * NP; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = base_n + nt * 8 + 2 * tid4 + (j & 1);
          s[nt][j] = n <= row_pos[j >> 1] ? fast_sigmoid(fmaf(s[nt][j], scale, row_bias[j >> 1])) : 0.f;
        }
#pragma unroll
      for (int kk = 0; kk < NP; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dt = 0; dt < KT; ++dt) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vt_s + (key0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + dt * 16 +
                                    (lane >> 4) * 8);
          mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
          mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
        }
      }
      __syncthreads();  // this stage may be overwritten by the load issued in the next iteration
    }
    cp_async_wait<0>();
  }

  if (!DECODE) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int R = row0 + warp_row + gid + 8 * r;
      if (R >= total_rows) continue;
      const int t = qs + R / g, head = hk * g + R % g;
      const float gt = gate ? gate[(size_t)t * Hq + head] : 1.f;
      __nv_bfloat16* dst = out + ((size_t)t * Hq + head) * D + 2 * tid4;
#pragma unroll
      for (int nt = 0; nt < 2 * KT; ++nt)
        *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) = __floats2bfloat162_rn(o[nt][2 * r] * gt, o[nt][2 * r + 1] * gt);
    }
    return;
  }
  // decode: the warps' sums of their keys are added in warp order
  __syncthreads();  // every warp is done with the tiles: shared memory becomes the reduction buffer
  float* red = reinterpret_cast<float*>(smem_raw);  // [warp][16][D + 1]
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int nt = 0; nt < 2 * KT; ++nt) {
      float* dst = red + ((size_t)warp * 16 + gid + 8 * r) * (D + 1) + nt * 8 + 2 * tid4;
      dst[0] = o[nt][2 * r];
      dst[1] = o[nt][2 * r + 1];
    }
  __syncthreads();
  for (int e = threadIdx.x; e < g * D; e += WARPS * 32) {
    const int rr = e / D, c = e % D;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += red[((size_t)w * 16 + rr) * (D + 1) + c];
    const int head = hk * g + rr;
    if (num_splits == 1) {
      const float gt = gate ? gate[(size_t)qs * Hq + head] : 1.f;
      out[((size_t)qs * Hq + head) * D + c] = __float2bfloat16_rn(v * gt);
    } else {
      partial[(((size_t)b * num_splits + blockIdx.x) * Hq + head) * D + c] = v;
    }
  }
}

// out[t(b), h, :] = gate * sum over the key ranges of partial[b, s, h, :], ranges in ascending order.
__global__ void sum_gate_kernel(const float* __restrict__ partial, const float* __restrict__ gate,
                                const int* __restrict__ q_start, __nv_bfloat16* __restrict__ out, int Hq, int D,
                                int num_splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, t = q_start[b];
  for (int e = threadIdx.x; e < Hq * D; e += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < num_splits; ++s) v += partial[((size_t)b * num_splits + s) * Hq * D + e];
    const float gt = gate ? gate[(size_t)t * Hq + e / D] : 1.f;
    out[(size_t)t * Hq * D + e] = __float2bfloat16_rn(v * gt);
  }
}

template <int KT, bool DECODE>
static int attn_sigmoid_mma_launch(const void* q, const void* k_pages, const void* v_pages, void* out, float* partial,
                                   const float* head_bias, const float* gate, const int* q_start, const int* kv_len,
                                   const int* block_table, int table_stride, int page_size, int num_pages, int B,
                                   int max_q_len, int Hq, int Hkv, float scale, int num_splits, int* status,
                                   cudaStream_t stream) {
  using S = SigmoidShape<KT, DECODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_sigmoid_mma_kernel<KT, DECODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)S::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int g = Hq / Hkv;
  const long long tiles = DECODE ? num_splits : ((long long)max_q_len * g + S::BM - 1) / S::BM;
  if (tiles > 0x7fffffffLL) return Q3_ERR_SIZE;
  dim3 grid((unsigned)tiles, Hkv, B);
  q3::launch(attn_sigmoid_mma_kernel<KT, DECODE>, dim3(grid), dim3(S::WARPS * 32), S::SMEM_BYTES, stream,
             (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out,
             partial, head_bias, gate, q_start, kv_len, block_table, table_stride, page_size, num_pages, Hq, Hkv, scale,
             num_splits, status);
  if (DECODE && num_splits > 1)
    q3::launch(sum_gate_kernel, dim3(B), dim3(256), 0, stream, (const float*)partial, gate, q_start, (__nv_bfloat16*)out,
               Hq, 16 * KT, num_splits);
  return launch_status();
}

}  // namespace q3

// q, out: bf16 [T, Hq, D]; pages: bf16 [num_pages, Hkv, page_size, D]; head_bias: float32 [Hq] or null; gate:
// float32 [T, Hq] or null.  decode != 0: the B sequences bring one token each (rows q_start[b]) and their keys
// are cut into num_splits ranges; partial: float32 [B, num_splits, Hq, D], needed for more than one range.
// Takes D in multiples of 16 up to 256 and, for decode, groups of up to 16 heads; refuses the rest.
extern "C" int q3_attn_sigmoid_mma(const void* q, const void* k_pages, const void* v_pages, void* out, float* partial,
                                   const float* head_bias, const float* gate, const int* q_start, const int* kv_len,
                                   const int* block_table, int table_stride, int page_size, int num_pages, int B,
                                   int max_q_len, int Hq, int Hkv, int D, float scale, int decode, int num_splits,
                                   int* status, cudaStream_t stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || D % 16 || D < 16 || D > 256 || page_size <= 0 || table_stride <= 0 || B > 65535 ||
      Hkv > 65535 || num_splits < 1 || (decode && Hq / Hkv > 16))
    return Q3_ERR_SIZE;
  if (decode && num_splits > 1 && !partial) return Q3_ERR_SCRATCH;
  if ((uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16 || (uintptr_t)out % 4) return Q3_ERR_ALIGN;
#define Q3_SM_CASE(KT)                                                                                              \
  case KT:                                                                                                          \
    if (decode)                                                                                                     \
      return q3::attn_sigmoid_mma_launch<KT, true>(q, k_pages, v_pages, out, partial, head_bias, gate, q_start, kv_len, \
                                                   block_table, table_stride, page_size, num_pages, B, 1, Hq, Hkv, scale, \
                                                   num_splits, status, stream);                                     \
    return q3::attn_sigmoid_mma_launch<KT, false>(q, k_pages, v_pages, out, nullptr, head_bias, gate, q_start, kv_len,  \
                                                  block_table, table_stride, page_size, num_pages, B, max_q_len, Hq, Hkv, \
                                                  scale, 1, status, stream);
  switch (D / 16) {
    Q3_SM_CASE(1) Q3_SM_CASE(2) Q3_SM_CASE(3) Q3_SM_CASE(4) Q3_SM_CASE(5) Q3_SM_CASE(6) Q3_SM_CASE(7) Q3_SM_CASE(8)
    Q3_SM_CASE(9) Q3_SM_CASE(10) Q3_SM_CASE(11) Q3_SM_CASE(12) Q3_SM_CASE(13) Q3_SM_CASE(14) Q3_SM_CASE(15)
    Q3_SM_CASE(16)
  }
#undef Q3_SM_CASE
  return Q3_ERR_SIZE;
}
