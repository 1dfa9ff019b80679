// Grouped-query attention over a sliding window of a paged key/value pool, with a softmax sink and per-head output
// gates, for a ragged in-flight batch; and the step in front of it that turns projected rows into queries and cache
// entries (short causal convolution -> rotation -> paged store).
//
// Pool entry of one position: [G][dim] rotated keys, then [G][vdim] values (G key/value heads).  Query head h reads
// key/value head h / (H / G).
//
//   qkv_conv_rope_append_kernel   one thread per (row, channel) of the concatenated q | k | v projection: the causal
//                                 convolution over the row's own portion and the sequence's carried inputs, the
//                                 rotation of the head's leading `dims` elements (interleaved pairs; the partner's
//                                 convolution is recomputed), and the store: queries to their buffer, keys and values
//                                 to the row's place in its sequence's pages.
//   window_attention_kernel       any sizes, fp32 or bf16: one CTA per (row, key/value head, 4 query heads of its group);
//                                 key blocks of 32 positions aligned to absolute positions, from the window's first block,
//                                 staged as fp32; lane = key for the scores, lane = value column for the weighted sum.
//   window_attention_mma_kernel   bf16, 16 | dim, 8 | vdim: one CTA per (sequence, key/value head, 16 / group-size query
//                                 positions ...) — see below.
//
// The softmax runs online in fp32 and starts from the sink: m = sink_h, l = 1, no value — so the sink is counted once,
// unscaled, whatever the number of key blocks.  Keys are visited in an order fixed by the row's position alone.
#include <cuda_bf16.h>

#include <cstdlib>

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

__device__ __forceinline__ float ld_w(const void* p, int dtype, int64_t i) {
  return dtype == TB_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

constexpr int kMaxTaps = 8;

struct QkvArgs {
  const float* proj; int64_t ldp;            // [rows, >= C] : q (H dim) | k (G dim) | v (G vdim)
  const void* conv_w; int w_dtype;           // [C, taps]
  const float* state;                        // [slots, taps - 1, C] carried inputs, oldest first
  const float* table;                        // [rows, dims / 2, 2] cos, sin
  const int *tok_seq, *tok_pos, *seq_start, *seq_past, *seq_slot, *block_table;
  int max_blocks, page, rows, H, G, dim, vdim, dims, taps;
};

// convolution output of channel ch at the row's position
__device__ __forceinline__ float conv_at(const QkvArgs& a, const float* st, int C, int ch, int pos, int past, int start) {
  float acc = 0.f;
  for (int k = 0; k < a.taps; ++k) {
    const int p = pos - (a.taps - 1 - k);
    float v = 0.f;
    if (p >= past) v = a.proj[(int64_t) (start + (p - past)) * a.ldp + ch];
    else if (p >= 0) v = st[(int64_t) (a.taps - 1 - (past - p)) * C + ch];     // state row j holds position past - (taps-1) + j
    acc = fmaf(ld_w(a.conv_w, a.w_dtype, (int64_t) ch * a.taps + k), v, acc);
  }
  return acc;
}

template <typename T>
__global__ void qkv_conv_rope_append_kernel(T* q_out, T* pool, QkvArgs a) {
  const int Cq = a.H * a.dim, Ck = a.G * a.dim, Cv = a.G * a.vdim, C = Cq + Ck + Cv;
  const int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x;
  if (i >= (int64_t) a.rows * C) return;
  const int row = (int) (i / C), ch = (int) (i % C);
  const int e = a.tok_seq[row], pos = a.tok_pos[row], past = a.seq_past[e], start = a.seq_start[e];
  const float* st = a.state + (int64_t) a.seq_slot[e] * (a.taps - 1) * C;
  float y = conv_at(a, st, C, ch, pos, past, start);
  if (ch < Cq + Ck) {
    const int d = (ch < Cq ? ch : ch - Cq) % a.dim;
    if (d < a.dims) {
      const float yp = conv_at(a, st, C, ch ^ 1, pos, past, start);      // dim-aligned pairs: heads start at even channels
      const float* cs = a.table + ((int64_t) row * (a.dims / 2) + d / 2) * 2;
      y = (d & 1) ? fmaf(y, cs[0], yp * cs[1]) : fmaf(y, cs[0], -yp * cs[1]);
    }
  }
  if (ch < Cq) {
    q_out[(int64_t) row * Cq + ch] = from_f<T>(y);
  } else {
    const int64_t slot = (int64_t) a.block_table[(int64_t) e * a.max_blocks + pos / a.page] * a.page + pos % a.page;
    pool[slot * (Ck + Cv) + (ch - Cq)] = from_f<T>(y);
  }
}

constexpr int kWarps = 4;
constexpr int kTile = 32;
constexpr int kMaxVPerLane = 8;          // vdim <= 256

struct AttnArgs {
  const float* gate; int64_t ldg;          // gate logits [rows, >= H] or NULL
  const void* sink; int sink_dtype;        // [H] or NULL
  const int *tok_seq, *tok_pos, *block_table;
  int max_blocks, page, H, G, dim, vdim, window;
  float scale;
};

// shared memory (fp32): keys [32][dim + 1] | values [32][vdim] | per warp q [dim]
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) window_attention_kernel(T* out, const T* q, const T* pool, AttnArgs a) {
  extern __shared__ float smem[];
  const int LDK = a.dim + 1, E = a.G * (a.dim + a.vdim), per = a.H / a.G;
  float* keys = smem;
  float* vals = keys + kTile * LDK;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  float* qs = vals + kTile * a.vdim + warp * a.dim;
  const int row = blockIdx.x, g = blockIdx.y;
  const int hl = blockIdx.z * kWarps + warp;            // head within the group
  const bool live = hl < per;
  const int head = g * per + (live ? hl : 0);
  const int pos = a.tok_pos[row];
  const int* bt = a.block_table + (int64_t) a.tok_seq[row] * a.max_blocks;
  const int lo = a.window > 0 && pos - a.window + 1 > 0 ? pos - a.window + 1 : 0;      // first visible position
  if (live) {
    const T* qsrc = q + ((int64_t) row * a.H + head) * a.dim;
    for (int d = lane; d < a.dim; d += 32) qs[d] = to_f<T>(qsrc[d]) * a.scale;
  }
  float acc[kMaxVPerLane];
#pragma unroll
  for (int c = 0; c < kMaxVPerLane; ++c) acc[c] = 0.f;
  float m = -INFINITY, l = 0.f;
  if (a.sink) { m = ld_w(a.sink, a.sink_dtype, head); l = 1.f; }
  for (int j0 = (lo / kTile) * kTile; j0 <= pos; j0 += kTile) {
    __syncthreads();
    for (int e = threadIdx.x; e < kTile * a.dim; e += kWarps * 32) {
      const int jj = e / a.dim, d = e % a.dim, j = j0 + jj;
      float v = 0.f;
      if (j >= lo && j <= pos) v = to_f<T>(pool[((int64_t) bt[j / a.page] * a.page + j % a.page) * E + g * a.dim + d]);
      keys[jj * LDK + d] = v;
    }
    for (int e = threadIdx.x; e < kTile * a.vdim; e += kWarps * 32) {
      const int jj = e / a.vdim, d = e % a.vdim, j = j0 + jj;
      float v = 0.f;
      if (j >= lo && j <= pos)
        v = to_f<T>(pool[((int64_t) bt[j / a.page] * a.page + j % a.page) * E + a.G * a.dim + g * a.vdim + d]);
      vals[jj * a.vdim + d] = v;
    }
    __syncthreads();
    if (!live) continue;
    float s = 0.f;
    const float* kr = keys + lane * LDK;
    for (int d = 0; d < a.dim; ++d) s = fmaf(qs[d], kr[d], s);
    const bool vis = j0 + lane >= lo && j0 + lane <= pos;
    s = vis ? s : -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));          // finite: every visited block holds a visible key
    const float p = vis ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);                 // 0 when m is still -inf
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) {
      const int col = c * 32 + lane;
      if (c * 32 >= a.vdim) break;                      // uniform over the warp
      const int cc = col < a.vdim ? col : a.vdim - 1;
      float v = acc[c] * corr;
#pragma unroll 8
      for (int jj = 0; jj < kTile; ++jj) v = fmaf(__shfl_sync(0xffffffffu, p, jj), vals[jj * a.vdim + cc], v);
      acc[c] = v;
    }
  }
  if (live) {
    float f = 1.f / l;
    if (a.gate) f *= 1.f / (1.f + expf(-a.gate[(int64_t) row * a.ldg + head]));
    T* dst = out + ((int64_t) row * a.H + head) * a.vdim;
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) {
      const int col = c * 32 + lane;
      if (col < a.vdim) dst[col] = from_f<T>(acc[c] * f);
    }
  }
}

}  // namespace
}  // namespace tb

using namespace tb;

extern "C" int tb_qkv_conv_rope_append(void* q_out, void* pool, int dtype, const float* proj, int64_t ldp, const void* conv_w,
                                       int w_dtype, const float* state, const float* table, int dims, const int* tok_seq,
                                       const int* tok_pos, const int* seq_start, const int* seq_past, const int* seq_slot,
                                       const int* block_table, int max_blocks, int page, int rows, int heads, int kv_heads,
                                       int dim, int vdim, int taps, tb_stream_t stream) {
  if (!q_out || !pool || !proj || !conv_w || !tok_seq || !tok_pos || !seq_start || !seq_past || !seq_slot || !block_table)
    return -1;
  if ((dtype != TB_DT_F32 && dtype != TB_DT_BF16) || (w_dtype != TB_DT_F32 && w_dtype != TB_DT_BF16)) return -1;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || taps < 1 || taps > kMaxTaps || page <= 0 ||
      rows < 0 || dims < 0 || dims % 2 || dims > dim || (dims > 0 && (dim % 2 || !table)) || (taps > 1 && !state))
    return -1;
  if (rows == 0) return 0;
  QkvArgs a{proj, ldp, conv_w, w_dtype, state, table, tok_seq, tok_pos, seq_start, seq_past, seq_slot, block_table,
            max_blocks, page, rows, heads, kv_heads, dim, vdim, dims, taps};
  const int64_t n = (int64_t) rows * ((int64_t) heads * dim + (int64_t) kv_heads * (dim + vdim));
  const unsigned grid = (unsigned) ((n + 255) / 256);
  if (dtype == TB_DT_F32) qkv_conv_rope_append_kernel<float><<<grid, 256, 0, (cudaStream_t) stream>>>((float*) q_out, (float*) pool, a);
  else qkv_conv_rope_append_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t) stream>>>((__nv_bfloat16*) q_out, (__nv_bfloat16*) pool, a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_window_attention_tensor_cores(int dtype, int heads, int kv_heads, int dim, int vdim) {
  (void) dtype; (void) heads; (void) kv_heads; (void) dim; (void) vdim;
  return 0;
}

extern "C" int tb_window_attention(void* out, const void* q, const void* pool, int dtype, const float* gate, int64_t ldg,
                                   const void* sink, int sink_dtype, const int* tok_seq, const int* tok_pos,
                                   const int* block_table, int max_blocks, int page, int rows, int heads, int kv_heads,
                                   int dim, int vdim, float scale, int window, int mode, tb_stream_t stream) {
  if (!out || !q || !pool || !tok_seq || !tok_pos || !block_table) return -1;
  if (dtype != TB_DT_F32 && dtype != TB_DT_BF16) return -1;
  if (sink && sink_dtype != TB_DT_F32 && sink_dtype != TB_DT_BF16) return -1;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || vdim > 32 * kMaxVPerLane || page <= 0 ||
      rows < 0 || window < 0 || kv_heads > 65535)
    return -1;
  if (rows == 0) return 0;
  AttnArgs a{gate, ldg, sink, sink_dtype, tok_seq, tok_pos, block_table, max_blocks, page, heads, kv_heads, dim, vdim,
             window, scale};
  const size_t smem = ((size_t) kTile * (dim + 1) + (size_t) kTile * vdim + (size_t) kWarps * dim) * sizeof(float);
  if (smem > 220 * 1024) return -2;
  dim3 grid(rows, kv_heads, (heads / kv_heads + kWarps - 1) / kWarps);
  cudaStream_t s = (cudaStream_t) stream;
  static size_t raised_f = 48 * 1024, raised_b = 48 * 1024;
  if (dtype == TB_DT_F32) {
    if (smem > raised_f) {
      TB_CHECK_CUDA(cudaFuncSetAttribute(window_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
      raised_f = smem;
    }
    window_attention_kernel<float><<<grid, kWarps * 32, smem, s>>>((float*) out, (const float*) q, (const float*) pool, a);
  } else {
    if (smem > raised_b) {
      TB_CHECK_CUDA(cudaFuncSetAttribute(window_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
      raised_b = smem;
    }
    window_attention_kernel<__nv_bfloat16><<<grid, kWarps * 32, smem, s>>>((__nv_bfloat16*) out, (const __nv_bfloat16*) q,
                                                                             (const __nv_bfloat16*) pool, a);
  }
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
