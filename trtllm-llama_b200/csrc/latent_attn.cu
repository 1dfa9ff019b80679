// Latent (compressed-KV) attention over a paged pool, for a ragged in-flight batch.
//
// The cache holds ONE entry per position and layer: the normalised latent c (lat values) followed by the rotated key
// part shared by all heads (rot_dim values).  Keys and values of the heads are linear images of c, so the kernels never
// materialise them: the query of a head arrives already multiplied by that head's key up-projection ("absorbed"), the
// score is a dot product with the cache entry itself, and the softmax-weighted sum of latents goes back through the
// head's value up-projection outside (tb_linear, batched over heads).  That makes this a multi-query attention with head
// size lat + rot_dim and value size lat, and decode reads (lat + rot_dim) elements per cached position instead of
// heads * (dim + vdim).
//
//   latent_kv_append_kernel   RMS norm of the latent + rotation of the key part + paged store, one warp per row
//   latent_attention_kernel   one CTA per (row, group of 4 heads); keys visited in blocks of 32 positions from 0,
//                             staged in shared memory as fp32 for the group; lane = key for the scores, lane = latent
//                             column for the weighted sum; online softmax in fp32
#include <cuda_bf16.h>

#include "common.cuh"
#include "../../include/trtllm_b200_ragged.h"

namespace tb {
namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float ld_w(const void* p, int dtype, int i) {
  return dtype == TB_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

template <typename T>
__global__ void __launch_bounds__(128) latent_kv_append_kernel(T* pool, const float* kv, int64_t ldkv, const void* w,
                                                               int w_dtype, float eps, const float* table, int dims,
                                                               const int* tok_seq, const int* tok_pos,
                                                               const int* block_table, int max_blocks, int page, int rows,
                                                               int lat, int rot_dim) {
  const int row = blockIdx.x * 4 + threadIdx.x / 32, lane = threadIdx.x % 32;
  if (row >= rows) return;
  const float* src = kv + (int64_t) row * ldkv;
  const int pos = tok_pos[row];
  const int blk = block_table[(int64_t) tok_seq[row] * max_blocks + pos / page];
  T* dst = pool + ((int64_t) blk * page + pos % page) * (lat + rot_dim);
  float ss = 0.f;
  for (int c = lane; c < lat; c += 32) ss = fmaf(src[c], src[c], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float) lat + eps);
  for (int c = lane; c < lat; c += 32) dst[c] = from_f<T>(src[c] * inv * ld_w(w, w_dtype, c));
  const float* kr = src + lat;
  for (int e = lane; e < rot_dim - dims / 2; e += 32) {
    if (e < dims / 2) {
      const float c = table[((int64_t) row * (dims / 2) + e) * 2], s = table[((int64_t) row * (dims / 2) + e) * 2 + 1];
      const float u = kr[2 * e], v = kr[2 * e + 1];
      dst[lat + 2 * e] = from_f<T>(u * c - v * s);
      dst[lat + 2 * e + 1] = from_f<T>(v * c + u * s);
    } else {
      const int j = dims + (e - dims / 2);
      dst[lat + j] = from_f<T>(kr[j]);
    }
  }
}

constexpr int kAttnWarps = 4;
constexpr int kKeyTile = 32;

// shared memory: keys [32][D + 1] | per warp: q [D], acc [lat]
template <typename T>
__global__ void __launch_bounds__(kAttnWarps * 32) latent_attention_kernel(T* out, const T* qa, const T* pool,
                                                                            const int* tok_seq, const int* tok_pos,
                                                                            const int* block_table, int max_blocks, int page,
                                                                            int heads, int lat, int rot_dim, float scale) {
  extern __shared__ float smem[];
  const int D = lat + rot_dim, LDK = D + 1;
  float* keys = smem;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  float* qs = smem + kKeyTile * LDK + warp * (D + lat);
  float* acc = qs + D;
  const int row = blockIdx.x;
  const int head = blockIdx.y * kAttnWarps + warp;
  const bool live = head < heads;
  const int pos = tok_pos[row];
  const int* bt = block_table + (int64_t) tok_seq[row] * max_blocks;
  if (live) {
    const T* qsrc = qa + ((int64_t) row * heads + head) * D;
    for (int d = lane; d < D; d += 32) qs[d] = to_f<T>(qsrc[d]) * scale;
    for (int c = lane; c < lat; c += 32) acc[c] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int j0 = 0; j0 <= pos; j0 += kKeyTile) {
    __syncthreads();                                  // the previous tile has been consumed (and qs / acc are written)
    for (int e = threadIdx.x; e < kKeyTile * D; e += kAttnWarps * 32) {
      const int jj = e / D, d = e % D, j = j0 + jj;
      float v = 0.f;
      if (j <= pos) v = to_f<T>(pool[((int64_t) bt[j / page] * page + j % page) * D + d]);
      keys[jj * LDK + d] = v;
    }
    __syncthreads();
    if (!live) continue;
    float s = 0.f;
    const float* kr = keys + lane * LDK;
    for (int d = 0; d < D; ++d) s = fmaf(qs[d], kr[d], s);
    const bool vis = j0 + lane <= pos;
    s = vis ? s : -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));        // finite: position j0 of every tile is visible
    const float p = vis ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);               // 0 on the first tile (m = -inf)
    l = l * corr + warp_sum(p);
    m = m_new;
    for (int c = lane; c < lat; c += 32) {
      float a = acc[c] * corr;
#pragma unroll 8
      for (int jj = 0; jj < kKeyTile; ++jj) a = fmaf(__shfl_sync(0xffffffffu, p, jj), keys[jj * LDK + c], a);
      acc[c] = a;
    }
  }
  if (live) {
    const float inv = 1.f / l;
    T* dst = out + ((int64_t) row * heads + head) * lat;
    for (int c = lane; c < lat; c += 32) dst[c] = from_f<T>(acc[c] * inv);
  }
}

}  // namespace
}  // namespace tb

using namespace tb;

extern "C" int tb_latent_kv_append(void* pool, int dtype, const float* kv, int64_t ldkv, const void* w, int w_dtype, float eps,
                                   const float* table, int dims, const int* tok_seq, const int* tok_pos,
                                   const int* block_table, int max_blocks, int page, int rows, int lat, int rot_dim,
                                   tb_stream_t stream) {
  if (!pool || !kv || !w || !table || !tok_seq || !tok_pos || !block_table || lat <= 0 || rot_dim <= 0 || dims <= 0 ||
      dims % 2 || dims > rot_dim || page <= 0 || max_blocks <= 0 || rows < 0)
    return -1;
  if ((dtype != TB_DT_F32 && dtype != TB_DT_BF16) || (w_dtype != TB_DT_F32 && w_dtype != TB_DT_BF16)) return -1;
  if (rows == 0) return 0;
  cudaStream_t s = (cudaStream_t) stream;
  const int grid = (rows + 3) / 4;
  if (dtype == TB_DT_F32)
    latent_kv_append_kernel<float><<<grid, 128, 0, s>>>((float*) pool, kv, ldkv, w, w_dtype, eps, table, dims, tok_seq,
                                                        tok_pos, block_table, max_blocks, page, rows, lat, rot_dim);
  else
    latent_kv_append_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>((__nv_bfloat16*) pool, kv, ldkv, w, w_dtype, eps, table, dims,
                                                                tok_seq, tok_pos, block_table, max_blocks, page, rows, lat,
                                                                rot_dim);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_latent_attention(void* out, const void* qa, const void* pool, int dtype, const int* tok_seq,
                                   const int* tok_pos, const int* block_table, int max_blocks, int page, int rows, int heads,
                                   int lat, int rot_dim, float scale, tb_stream_t stream) {
  if (!out || !qa || !pool || !tok_seq || !tok_pos || !block_table || heads <= 0 || lat <= 0 || rot_dim < 0 || page <= 0 ||
      max_blocks <= 0 || rows < 0)
    return -1;
  if (dtype != TB_DT_F32 && dtype != TB_DT_BF16) return -1;
  if (rows == 0) return 0;
  const int D = lat + rot_dim;
  const size_t smem = sizeof(float) * ((size_t) kKeyTile * (D + 1) + (size_t) kAttnWarps * (D + lat));
  if (smem > 227 * 1024) return -2;
  cudaStream_t s = (cudaStream_t) stream;
  dim3 grid(rows, (heads + kAttnWarps - 1) / kAttnWarps);
  if (dtype == TB_DT_F32) {
    TB_CHECK_CUDA(cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    latent_attention_kernel<float><<<grid, kAttnWarps * 32, smem, s>>>((float*) out, (const float*) qa, (const float*) pool,
                                                                       tok_seq, tok_pos, block_table, max_blocks, page, heads,
                                                                       lat, rot_dim, scale);
  } else {
    TB_CHECK_CUDA(cudaFuncSetAttribute(latent_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int) smem));
    latent_attention_kernel<__nv_bfloat16><<<grid, kAttnWarps * 32, smem, s>>>(
        (__nv_bfloat16*) out, (const __nv_bfloat16*) qa, (const __nv_bfloat16*) pool, tok_seq, tok_pos, block_table,
        max_blocks, page, heads, lat, rot_dim, scale);
  }
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
