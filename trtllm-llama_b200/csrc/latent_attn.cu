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
    for (int c0 = 0; c0 < lat; c0 += 32) {            // every lane takes every trip: the shuffles below need the whole warp
      const int c = c0 + lane < lat ? c0 + lane : lat - 1;
      float a = acc[c] * corr;
#pragma unroll 8
      for (int jj = 0; jj < kKeyTile; ++jj) a = fmaf(__shfl_sync(0xffffffffu, p, jj), keys[jj * LDK + c], a);
      __syncwarp();
      if (c0 + lane < lat) acc[c] = a;
      __syncwarp();
    }
  }
  if (live) {
    const float inv = 1.f / l;
    T* dst = out + ((int64_t) row * heads + head) * lat;
    for (int c = lane; c < lat; c += 32) dst[c] = from_f<T>(acc[c] * inv);
  }
}


// ---------------------------------------------------------------------------------------------------------------
// Tensor-core form (bf16 storage): one CTA = one query row x 16 heads (the MMA's M) x one range of key tiles.
//   S [16 x 32]  = Q [16 x D] . K^T          warp w owns keys 8w..8w+7 of the tile (mma.sync m16n8k16, fp32 accumulators)
//   softmax      row maxima / sums exchanged through shared memory, fp32, every warp keeps the same running (m, l)
//   O [16 x lat] += P [16 x 32] . C          warp w owns latent columns [w lat/4, (w+1) lat/4); the B fragments come out of
//                                            the row-major key tile with ldmatrix.trans, so the tile is staged once and
//                                            serves as K and as V
// Key tiles arrive through a two-stage cp.async ring (16-byte copies, zero-filled past the row's position, so nothing
// uninitialised in the pool can reach an accumulator).  With nsplit > 1 (few rows, long contexts: decoding) the key tiles
// are dealt to nsplit CTAs per (row, head group) whose unnormalised partial results are merged by a second kernel.
constexpr int kTcHeads = 16;
constexpr int kPsLd = kKeyTile + 8;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
  const uint32_t d = (uint32_t) __cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <int NTO>   // n8 tiles of the latent per warp: lat = 32 * NTO
__global__ void __launch_bounds__(128) latent_attention_mma_kernel(__nv_bfloat16* out, float* partial, const __nv_bfloat16* qa,
                                                                   const __nv_bfloat16* pool, const int* tok_seq,
                                                                   const int* tok_pos, const int* block_table, int max_blocks,
                                                                   int page, int heads, int rot_dim, float scale, int nsplit) {
  constexpr int LAT = NTO * 32;
  const int D = LAT + rot_dim, LDK = D + 8, CH = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [16][LDK]
  __nv_bfloat16* Ks = Qs + kTcHeads * LDK;                             // [2][32][LDK]
  __nv_bfloat16* Ps = Ks + 2 * kKeyTile * LDK;                         // [16][40]
  float* red = reinterpret_cast<float*>(Ps + kTcHeads * kPsLd);        // [2][4][16]: row maxima, row sums per warp
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32, g = lane / 4, t = lane % 4;
  const int row = blockIdx.x, hg = blockIdx.y, split = blockIdx.z;
  const int pos = tok_pos[row];
  const int* bt = block_table + (int64_t) tok_seq[row] * max_blocks;
  const int tiles_total = pos / kKeyTile + 1;
  const int per = (tiles_total + nsplit - 1) / nsplit;
  const int t0 = split * per, t1 = min(tiles_total, t0 + per);
  const int page_shift = 31 - __clz(page), page_mask = page - 1;        // pages are powers of two (checked by the launcher)

  for (int e = tid; e < kTcHeads * CH; e += 128) {
    const int r = e / CH, c = e % CH, head = hg * kTcHeads + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (head < heads) v = *reinterpret_cast<const uint4*>(qa + ((int64_t) row * heads + head) * D + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * LDK + c * 8) = v;
  }
  // a warp copies every fourth key of the tile, its lanes the 16-byte pieces of the entry: no divisions, one table
  // lookup per key
  auto load_tile = [&](int tile, int buf) {
    const int j0 = tile * kKeyTile;
    for (int jj = warp; jj < kKeyTile; jj += 4) {
      const int j = j0 + jj;
      const bool ok = j <= pos;
      const __nv_bfloat16* src = ok ? pool + (((int64_t) bt[j >> page_shift] << page_shift) + (j & page_mask)) * D : pool;
      __nv_bfloat16* dst = Ks + (buf * kKeyTile + jj) * LDK;
      for (int c = lane; c < CH; c += 32) cp_async16(dst + c * 8, ok ? src + c * 8 : src, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[NTO][4];
#pragma unroll
  for (int n = 0; n < NTO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  if (t0 < t1) load_tile(t0, 0);
  for (int tile = t0; tile < t1; ++tile) {
    const int buf = (tile - t0) & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();        // this tile is in shared memory, and every warp is done with the previous one:
    if (tile + 1 < t1) load_tile(tile + 1, buf ^ 1);      // its buffer, the P tile and the maxima can be written again
    const __nv_bfloat16* Kb = Ks + buf * kKeyTile * LDK;
    float s[4];
    {
      // four accumulators take the k steps in turn: a chain of D / 16 dependent MMAs would leave the tensor pipe idle
      float sp[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) sp[i][0] = sp[i][1] = sp[i][2] = sp[i][3] = 0.f;
      // fragments come through ldmatrix: one instruction per 16 x 16 query block, one per two k steps of the keys.
      // A block: matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15); B: keys 8w..8w+7 x four runs of 8 k
      const int mi = lane >> 3, r8 = lane & 7;
      const uint32_t q_addr = (uint32_t) __cvta_generic_to_shared(Qs + (r8 + (mi & 1) * 8) * LDK + (mi >> 1) * 8);
      const uint32_t k_addr = (uint32_t) __cvta_generic_to_shared(Kb + (warp * 8 + r8) * LDK + mi * 8);
      int kk = 0;
      for (; kk + 64 <= D; kk += 64) {
        uint32_t a0[4], a1[4], a2[4], a3[4], b01[4], b23[4];
        ldsm_x4(a0, q_addr + kk * 2);
        ldsm_x4(a1, q_addr + (kk + 16) * 2);
        ldsm_x4(a2, q_addr + (kk + 32) * 2);
        ldsm_x4(a3, q_addr + (kk + 48) * 2);
        ldsm_x4(b01, k_addr + kk * 2);
        ldsm_x4(b23, k_addr + (kk + 32) * 2);
        mma_bf16_16816(sp[0], a0, b01[0], b01[1]);
        mma_bf16_16816(sp[1], a1, b01[2], b01[3]);
        mma_bf16_16816(sp[2], a2, b23[0], b23[1]);
        mma_bf16_16816(sp[3], a3, b23[2], b23[3]);
      }
      for (; kk + 32 <= D; kk += 32) {
        uint32_t a0[4], a1[4], b01[4];
        ldsm_x4(a0, q_addr + kk * 2);
        ldsm_x4(a1, q_addr + (kk + 16) * 2);
        ldsm_x4(b01, k_addr + kk * 2);
        mma_bf16_16816(sp[0], a0, b01[0], b01[1]);
        mma_bf16_16816(sp[1], a1, b01[2], b01[3]);
      }
      if (kk < D) {          // one k step of 16 left (lanes 16-31 give valid, unused addresses)
        uint32_t a0[4], b0, b1;
        ldsm_x4(a0, q_addr + kk * 2);
        ldsm_x2(b0, b1, (uint32_t) __cvta_generic_to_shared(Kb + (warp * 8 + r8) * LDK + (mi & 1) * 8) + kk * 2);
        mma_bf16_16816(sp[2], a0, b0, b1);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = (sp[0][i] + sp[1][i]) + (sp[2][i] + sp[3][i]);
    }
    const int j = tile * kKeyTile + warp * 8 + 2 * t;
    s[0] = j <= pos ? s[0] * scale : -INFINITY;
    s[1] = j + 1 <= pos ? s[1] * scale : -INFINITY;
    s[2] = j <= pos ? s[2] * scale : -INFINITY;
    s[3] = j + 1 <= pos ? s[3] * scale : -INFINITY;
    float mx0 = fmaxf(s[0], s[1]), mx1 = fmaxf(s[2], s[3]);
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if (t == 0) { red[warp * 16 + g] = mx0; red[warp * 16 + g + 8] = mx1; }
    __syncthreads();
    float mn0 = m0, mn1 = m1;
#pragma unroll
    for (int w = 0; w < 4; ++w) { mn0 = fmaxf(mn0, red[w * 16 + g]); mn1 = fmaxf(mn1, red[w * 16 + g + 8]); }
    // mn finite: the tile's first key is visible to every row
    const __nv_bfloat162 p01 = __floats2bfloat162_rn(__expf(s[0] - mn0), __expf(s[1] - mn0));
    const __nv_bfloat162 p23 = __floats2bfloat162_rn(__expf(s[2] - mn1), __expf(s[3] - mn1));
    *reinterpret_cast<__nv_bfloat162*>(Ps + g * kPsLd + warp * 8 + 2 * t) = p01;
    *reinterpret_cast<__nv_bfloat162*>(Ps + (g + 8) * kPsLd + warp * 8 + 2 * t) = p23;
    // the row sums stay per thread (its two keys of the tile) until the end: every thread rescales by the same factor
    const float c0 = __expf(m0 - mn0), c1 = __expf(m1 - mn1);     // 0 on the first tile
    l0 = l0 * c0 + (__bfloat162float(p01.x) + __bfloat162float(p01.y));
    l1 = l1 * c1 + (__bfloat162float(p23.x) + __bfloat162float(p23.y));
    m0 = mn0;
    m1 = mn1;
    __syncthreads();        // the P tile is complete
#pragma unroll
    for (int n = 0; n < NTO; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
    {
      const int mi = lane >> 3, r8 = lane & 7;
      const uint32_t p_addr = (uint32_t) __cvta_generic_to_shared(Ps + (r8 + (mi & 1) * 8) * kPsLd + (mi >> 1) * 8);
      // V fragments: the key tile itself, transposed on the way in; one ldmatrix.x4 feeds two 8-column tiles
      const uint32_t v_addr = (uint32_t) __cvta_generic_to_shared(Kb + (r8 + (mi & 1) * 8) * LDK + warp * (LAT / 4) + (mi >> 1) * 8);
#pragma unroll
      for (int kk = 0; kk < kKeyTile; kk += 16) {
        uint32_t a[4];
        ldsm_x4(a, p_addr + kk * 2);
        const uint32_t vk = v_addr + kk * LDK * 2;
#pragma unroll
        for (int n = 0; n + 1 < NTO; n += 2) {
          uint32_t b[4];
          ldsm_x4_trans(b, vk + n * 16);
          mma_bf16_16816(o[n], a, b[0], b[1]);
          mma_bf16_16816(o[n + 1], a, b[2], b[3]);
        }
        if (NTO & 1) {
          uint32_t b0, b1;
          const uint32_t kaddr = (uint32_t) __cvta_generic_to_shared(Kb + (kk + (lane & 15)) * LDK + warp * (LAT / 4)) + (NTO - 1) * 16;
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(kaddr));
          mma_bf16_16816(o[NTO - 1], a, b0, b1);
        }
      }
    }
  }
  // row sums: over the four threads of a row group, then over the warps (each saw its own keys of every tile)
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();
  if (t == 0) { red[64 + warp * 16 + g] = l0; red[64 + warp * 16 + g + 8] = l1; }
  __syncthreads();
  l0 = (red[64 + g] + red[64 + 16 + g]) + (red[64 + 32 + g] + red[64 + 48 + g]);
  l1 = (red[64 + g + 8] + red[64 + 16 + g + 8]) + (red[64 + 32 + g + 8] + red[64 + 48 + g + 8]);

  const int h0 = hg * kTcHeads + g, h1 = h0 + 8;
  if (nsplit == 1) {
    const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
    for (int n = 0; n < NTO; ++n) {
      const int col = warp * (LAT / 4) + n * 8 + 2 * t;
      if (h0 < heads)
        *reinterpret_cast<__nv_bfloat162*>(out + ((int64_t) row * heads + h0) * LAT + col) = __floats2bfloat162_rn(o[n][0] * i0, o[n][1] * i0);
      if (h1 < heads)
        *reinterpret_cast<__nv_bfloat162*>(out + ((int64_t) row * heads + h1) * LAT + col) = __floats2bfloat162_rn(o[n][2] * i1, o[n][3] * i1);
    }
  } else {
    // partial [row][head][split][LAT + 2]: unnormalised sums, then the running maximum and the running sum
#pragma unroll
    for (int n = 0; n < NTO; ++n) {
      const int col = warp * (LAT / 4) + n * 8 + 2 * t;
      if (h0 < heads) {
        float* d = partial + (((int64_t) row * heads + h0) * nsplit + split) * (LAT + 2);
        d[col] = o[n][0]; d[col + 1] = o[n][1];
      }
      if (h1 < heads) {
        float* d = partial + (((int64_t) row * heads + h1) * nsplit + split) * (LAT + 2);
        d[col] = o[n][2]; d[col + 1] = o[n][3];
      }
    }
    if (warp == 0 && t == 0) {
      if (h0 < heads) { float* d = partial + (((int64_t) row * heads + h0) * nsplit + split) * (LAT + 2); d[LAT] = m0; d[LAT + 1] = l0; }
      if (h1 < heads) { float* d = partial + (((int64_t) row * heads + h1) * nsplit + split) * (LAT + 2); d[LAT] = m1; d[LAT + 1] = l1; }
    }
  }
}

// Eight-warp form for 64 | lat and 32 | (lat + rot): twice the warps per SM at the same shared memory.  Warps w and w + 4
// split the k range of the score product for keys 8w..8w+7 and add their halves through shared memory (fixed order);
// every warp owns lat / 8 output columns, so the output tile costs half the registers.
template <int NTO>   // lat = 32 * NTO, NTO even
__global__ void __launch_bounds__(256, 2) latent_attention_mma8_kernel(__nv_bfloat16* out, float* partial, const __nv_bfloat16* qa,
                                                                   const __nv_bfloat16* pool, const int* tok_seq,
                                                                   const int* tok_pos, const int* block_table, int max_blocks,
                                                                   int page, int heads, int rot_dim, float scale, int nsplit) {
  constexpr int LAT = NTO * 32;
  const int D = LAT + rot_dim, LDK = D + 8, CH = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [16][LDK]
  __nv_bfloat16* Ks = Qs + kTcHeads * LDK;                             // [2][32][LDK]
  __nv_bfloat16* Ps = Ks + 2 * kKeyTile * LDK;                         // [16][40]
  float* red = reinterpret_cast<float*>(Ps + kTcHeads * kPsLd);        // [2][4][16]: row maxima, row sums per warp
  float4* spart = reinterpret_cast<float4*>(red + 128);                // [2 halves][4 key groups][32 lanes]
  const int tid = threadIdx.x, warp8 = tid / 32, lane = tid % 32, g = lane / 4, t = lane % 4;
  const int warp = warp8 & 3, half = warp8 >> 2;       // key group of the tile, half of the k range
  const int row = blockIdx.x, hg = blockIdx.y, split = blockIdx.z;
  const int pos = tok_pos[row];
  const int* bt = block_table + (int64_t) tok_seq[row] * max_blocks;
  const int tiles_total = pos / kKeyTile + 1;
  const int per = (tiles_total + nsplit - 1) / nsplit;
  const int t0 = split * per, t1 = min(tiles_total, t0 + per);
  const int page_shift = 31 - __clz(page), page_mask = page - 1;        // pages are powers of two (checked by the launcher)

  for (int e = tid; e < kTcHeads * CH; e += 256) {
    const int r = e / CH, c = e % CH, head = hg * kTcHeads + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (head < heads) v = *reinterpret_cast<const uint4*>(qa + ((int64_t) row * heads + head) * D + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * LDK + c * 8) = v;
  }
  // a warp copies every fourth key of the tile, its lanes the 16-byte pieces of the entry: no divisions, one table
  // lookup per key
  auto load_tile = [&](int tile, int buf) {
    const int j0 = tile * kKeyTile;
    for (int jj = warp8; jj < kKeyTile; jj += 8) {
      const int j = j0 + jj;
      const bool ok = j <= pos;
      const __nv_bfloat16* src = ok ? pool + (((int64_t) bt[j >> page_shift] << page_shift) + (j & page_mask)) * D : pool;
      __nv_bfloat16* dst = Ks + (buf * kKeyTile + jj) * LDK;
      for (int c = lane; c < CH; c += 32) cp_async16(dst + c * 8, ok ? src + c * 8 : src, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  constexpr int NW = NTO / 2;          // n8 tiles of the output per warp
  float o[NW][4];
#pragma unroll
  for (int n = 0; n < NW; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  const int kbeg = half * (D / 2), kend = kbeg + D / 2;

  if (t0 < t1) load_tile(t0, 0);
  for (int tile = t0; tile < t1; ++tile) {
    const int buf = (tile - t0) & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();        // this tile is in shared memory, and every warp is done with the previous one:
    if (tile + 1 < t1) load_tile(tile + 1, buf ^ 1);      // its buffer, the P tile and the maxima can be written again
    const __nv_bfloat16* Kb = Ks + buf * kKeyTile * LDK;
    float s[4];
    {
      // four accumulators take the k steps in turn: a chain of D / 16 dependent MMAs would leave the tensor pipe idle
      float sp[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) sp[i][0] = sp[i][1] = sp[i][2] = sp[i][3] = 0.f;
      // fragments come through ldmatrix: one instruction per 16 x 16 query block, one per two k steps of the keys.
      // A block: matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15); B: keys 8w..8w+7 x four runs of 8 k
      const int mi = lane >> 3, r8 = lane & 7;
      const uint32_t q_addr = (uint32_t) __cvta_generic_to_shared(Qs + (r8 + (mi & 1) * 8) * LDK + (mi >> 1) * 8);
      const uint32_t k_addr = (uint32_t) __cvta_generic_to_shared(Kb + (warp * 8 + r8) * LDK + mi * 8);
      int kk = kbeg;
      for (; kk + 64 <= kend; kk += 64) {
        uint32_t a0[4], a1[4], a2[4], a3[4], b01[4], b23[4];
        ldsm_x4(a0, q_addr + kk * 2);
        ldsm_x4(a1, q_addr + (kk + 16) * 2);
        ldsm_x4(a2, q_addr + (kk + 32) * 2);
        ldsm_x4(a3, q_addr + (kk + 48) * 2);
        ldsm_x4(b01, k_addr + kk * 2);
        ldsm_x4(b23, k_addr + (kk + 32) * 2);
        mma_bf16_16816(sp[0], a0, b01[0], b01[1]);
        mma_bf16_16816(sp[1], a1, b01[2], b01[3]);
        mma_bf16_16816(sp[2], a2, b23[0], b23[1]);
        mma_bf16_16816(sp[3], a3, b23[2], b23[3]);
      }
      for (; kk + 32 <= kend; kk += 32) {
        uint32_t a0[4], a1[4], b01[4];
        ldsm_x4(a0, q_addr + kk * 2);
        ldsm_x4(a1, q_addr + (kk + 16) * 2);
        ldsm_x4(b01, k_addr + kk * 2);
        mma_bf16_16816(sp[0], a0, b01[0], b01[1]);
        mma_bf16_16816(sp[1], a1, b01[2], b01[3]);
      }
      if (kk < kend) {          // one k step of 16 left (lanes 16-31 give valid, unused addresses)
        uint32_t a0[4], b0, b1;
        ldsm_x4(a0, q_addr + kk * 2);
        ldsm_x2(b0, b1, (uint32_t) __cvta_generic_to_shared(Kb + (warp * 8 + r8) * LDK + (mi & 1) * 8) + kk * 2);
        mma_bf16_16816(sp[2], a0, b0, b1);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = (sp[0][i] + sp[1][i]) + (sp[2][i] + sp[3][i]);
      spart[(half * 4 + warp) * 32 + lane] = make_float4(s[0], s[1], s[2], s[3]);
      __syncthreads();
      const float4 lo = spart[warp * 32 + lane], hi = spart[(4 + warp) * 32 + lane];
      s[0] = lo.x + hi.x; s[1] = lo.y + hi.y; s[2] = lo.z + hi.z; s[3] = lo.w + hi.w;
    }
    const int j = tile * kKeyTile + warp * 8 + 2 * t;
    s[0] = j <= pos ? s[0] * scale : -INFINITY;
    s[1] = j + 1 <= pos ? s[1] * scale : -INFINITY;
    s[2] = j <= pos ? s[2] * scale : -INFINITY;
    s[3] = j + 1 <= pos ? s[3] * scale : -INFINITY;
    float mx0 = fmaxf(s[0], s[1]), mx1 = fmaxf(s[2], s[3]);
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if (t == 0 && half == 0) { red[warp * 16 + g] = mx0; red[warp * 16 + g + 8] = mx1; }
    __syncthreads();
    float mn0 = m0, mn1 = m1;
#pragma unroll
    for (int w = 0; w < 4; ++w) { mn0 = fmaxf(mn0, red[w * 16 + g]); mn1 = fmaxf(mn1, red[w * 16 + g + 8]); }
    // mn finite: the tile's first key is visible to every row
    const __nv_bfloat162 p01 = __floats2bfloat162_rn(__expf(s[0] - mn0), __expf(s[1] - mn0));
    const __nv_bfloat162 p23 = __floats2bfloat162_rn(__expf(s[2] - mn1), __expf(s[3] - mn1));
    if (half == 0) {
      *reinterpret_cast<__nv_bfloat162*>(Ps + g * kPsLd + warp * 8 + 2 * t) = p01;
      *reinterpret_cast<__nv_bfloat162*>(Ps + (g + 8) * kPsLd + warp * 8 + 2 * t) = p23;
    }
    // the row sums stay per thread (its two keys of the tile) until the end: every thread rescales by the same factor
    const float c0 = __expf(m0 - mn0), c1 = __expf(m1 - mn1);     // 0 on the first tile
    l0 = l0 * c0 + (__bfloat162float(p01.x) + __bfloat162float(p01.y));
    l1 = l1 * c1 + (__bfloat162float(p23.x) + __bfloat162float(p23.y));
    m0 = mn0;
    m1 = mn1;
    __syncthreads();        // the P tile is complete
#pragma unroll
    for (int n = 0; n < NW; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
    {
      const int mi = lane >> 3, r8 = lane & 7;
      const uint32_t p_addr = (uint32_t) __cvta_generic_to_shared(Ps + (r8 + (mi & 1) * 8) * kPsLd + (mi >> 1) * 8);
      // V fragments: the key tile itself, transposed on the way in; one ldmatrix.x4 feeds two 8-column tiles
      const uint32_t v_addr = (uint32_t) __cvta_generic_to_shared(Kb + (r8 + (mi & 1) * 8) * LDK + warp8 * (LAT / 8) + (mi >> 1) * 8);
#pragma unroll
      for (int kk = 0; kk < kKeyTile; kk += 16) {
        uint32_t a[4];
        ldsm_x4(a, p_addr + kk * 2);
        const uint32_t vk = v_addr + kk * LDK * 2;
#pragma unroll
        for (int n = 0; n + 1 < NW; n += 2) {
          uint32_t b[4];
          ldsm_x4_trans(b, vk + n * 16);
          mma_bf16_16816(o[n], a, b[0], b[1]);
          mma_bf16_16816(o[n + 1], a, b[2], b[3]);
        }
        if (NW & 1) {
          uint32_t b0, b1;
          const uint32_t kaddr = (uint32_t) __cvta_generic_to_shared(Kb + (kk + (lane & 15)) * LDK + warp8 * (LAT / 8)) + (NW - 1) * 16;
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(kaddr));
          mma_bf16_16816(o[NW - 1], a, b0, b1);
        }
      }
    }
  }
  // row sums: over the four threads of a row group, then over the warps (each saw its own keys of every tile)
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();
  if (t == 0 && half == 0) { red[64 + warp * 16 + g] = l0; red[64 + warp * 16 + g + 8] = l1; }
  __syncthreads();
  l0 = (red[64 + g] + red[64 + 16 + g]) + (red[64 + 32 + g] + red[64 + 48 + g]);
  l1 = (red[64 + g + 8] + red[64 + 16 + g + 8]) + (red[64 + 32 + g + 8] + red[64 + 48 + g + 8]);

  const int h0 = hg * kTcHeads + g, h1 = h0 + 8;
  if (nsplit == 1) {
    const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
    for (int n = 0; n < NW; ++n) {
      const int col = warp8 * (LAT / 8) + n * 8 + 2 * t;
      if (h0 < heads)
        *reinterpret_cast<__nv_bfloat162*>(out + ((int64_t) row * heads + h0) * LAT + col) = __floats2bfloat162_rn(o[n][0] * i0, o[n][1] * i0);
      if (h1 < heads)
        *reinterpret_cast<__nv_bfloat162*>(out + ((int64_t) row * heads + h1) * LAT + col) = __floats2bfloat162_rn(o[n][2] * i1, o[n][3] * i1);
    }
  } else {
    // partial [row][head][split][LAT + 2]: unnormalised sums, then the running maximum and the running sum
#pragma unroll
    for (int n = 0; n < NW; ++n) {
      const int col = warp8 * (LAT / 8) + n * 8 + 2 * t;
      if (h0 < heads) {
        float* d = partial + (((int64_t) row * heads + h0) * nsplit + split) * (LAT + 2);
        d[col] = o[n][0]; d[col + 1] = o[n][1];
      }
      if (h1 < heads) {
        float* d = partial + (((int64_t) row * heads + h1) * nsplit + split) * (LAT + 2);
        d[col] = o[n][2]; d[col + 1] = o[n][3];
      }
    }
    if (warp8 == 0 && t == 0) {
      if (h0 < heads) { float* d = partial + (((int64_t) row * heads + h0) * nsplit + split) * (LAT + 2); d[LAT] = m0; d[LAT + 1] = l0; }
      if (h1 < heads) { float* d = partial + (((int64_t) row * heads + h1) * nsplit + split) * (LAT + 2); d[LAT] = m1; d[LAT + 1] = l1; }
    }
  }
}

// one CTA per (row, head): out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M), splits in index order
__global__ void latent_attention_merge_kernel(__nv_bfloat16* out, const float* partial, int lat, int nsplit) {
  const int64_t rh = blockIdx.x;
  const float* p = partial + rh * nsplit * (lat + 2);
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, p[s * (lat + 2) + lat]);
  float L = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float l = p[s * (lat + 2) + lat + 1];
    if (l > 0.f) L += l * __expf(p[s * (lat + 2) + lat] - M);
  }
  const float inv = 1.f / L;
  for (int c = threadIdx.x; c < lat; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float l = p[s * (lat + 2) + lat + 1];
      if (l > 0.f) acc += p[s * (lat + 2) + c] * __expf(p[s * (lat + 2) + lat] - M);
    }
    out[rh * lat + c] = __float2bfloat16_rn(acc * inv);
  }
}

// TB_LATENT_ATTN_WARPS=4 keeps every shape on the four-warp kernel (A/B measurements)
static bool latent_attention_four_warps() {
  static const bool on = [] { const char* e = getenv("TB_LATENT_ATTN_WARPS"); return e && e[0] == '4'; }();
  return on;
}

template <int NTO>
int launch_latent_mma(__nv_bfloat16* out, float* partial, const __nv_bfloat16* qa, const __nv_bfloat16* pool, const int* tok_seq,
                      const int* tok_pos, const int* block_table, int max_blocks, int page, int rows, int heads, int rot_dim,
                      float scale, int nsplit, cudaStream_t s) {
  const int D = NTO * 32 + rot_dim;
  const size_t smem = (size_t) (kTcHeads + 2 * kKeyTile) * (D + 8) * 2 + kTcHeads * kPsLd * 2 + 2 * 4 * 16 * sizeof(float);
  if (smem > 227 * 1024) return -2;
  dim3 grid(rows, (heads + kTcHeads - 1) / kTcHeads, nsplit);
  if constexpr (NTO % 2 == 0) {
    if (D % 32 == 0 && !latent_attention_four_warps()) {
      const size_t smem8 = smem + 2 * 4 * 32 * sizeof(float4);
      static size_t raised8 = 48 * 1024;
      if (smem8 > raised8) {
        TB_CHECK_CUDA(cudaFuncSetAttribute(latent_attention_mma8_kernel<NTO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem8));
        raised8 = smem8;
      }
      latent_attention_mma8_kernel<NTO><<<grid, 256, smem8, s>>>(out, partial, qa, pool, tok_seq, tok_pos, block_table, max_blocks,
                                                                page, heads, rot_dim, scale, nsplit);
      TB_CHECK_CUDA(cudaGetLastError());
      if (nsplit > 1) {
        latent_attention_merge_kernel<<<rows * heads, 128, 0, s>>>(out, partial, NTO * 32, nsplit);
        TB_CHECK_CUDA(cudaGetLastError());
      }
      return 0;
    }
  }
  static size_t raised = 48 * 1024;      // the opt-in only ever grows, and only outside a replayed region
  if (smem > raised) {
    TB_CHECK_CUDA(cudaFuncSetAttribute(latent_attention_mma_kernel<NTO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    raised = smem;
  }
  latent_attention_mma_kernel<NTO><<<grid, 128, smem, s>>>(out, partial, qa, pool, tok_seq, tok_pos, block_table, max_blocks,
                                                           page, heads, rot_dim, scale, nsplit);
  TB_CHECK_CUDA(cudaGetLastError());
  if (nsplit > 1) {
    latent_attention_merge_kernel<<<rows * heads, 128, 0, s>>>(out, partial, NTO * 32, nsplit);
    TB_CHECK_CUDA(cudaGetLastError());
  }
  return 0;
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

extern "C" int tb_latent_attention_tensor_cores(int dtype, int lat, int rot_dim) {
  const int nto = lat / 32;
  const bool have = nto == 1 || nto == 2 || nto == 3 || nto == 4 || nto == 5 || nto == 6 || nto == 8 || nto == 12 || nto == 16;
  return dtype == TB_DT_BF16 && lat % 32 == 0 && have && rot_dim % 16 == 0;
}

extern "C" int tb_latent_attention(void* out, const void* qa, const void* pool, int dtype, const int* tok_seq,
                                   const int* tok_pos, const int* block_table, int max_blocks, int page, int rows, int heads,
                                   int lat, int rot_dim, float scale, int nsplit, float* workspace, tb_stream_t stream) {
  if (!out || !qa || !pool || !tok_seq || !tok_pos || !block_table || heads <= 0 || lat <= 0 || rot_dim < 0 || page <= 0 ||
      max_blocks <= 0 || rows < 0)
    return -1;
  if (dtype != TB_DT_F32 && dtype != TB_DT_BF16) return -1;
  if (rows == 0) return 0;
  if (nsplit >= 0 && tb_latent_attention_tensor_cores(dtype, lat, rot_dim) && (page & (page - 1)) == 0 && (uintptr_t) qa % 16 == 0 && (uintptr_t) pool % 16 == 0 &&
      (uintptr_t) out % 4 == 0) {
    if (nsplit < 1 || !workspace) nsplit = 1;
    if (nsplit > 64) nsplit = 64;
#define TB_LAT_CASE(n)                                                                                                   \
  case n:                                                                                                               \
    return launch_latent_mma<n>((__nv_bfloat16*) out, workspace, (const __nv_bfloat16*) qa, (const __nv_bfloat16*) pool, \
                                tok_seq, tok_pos, block_table, max_blocks, page, rows, heads, rot_dim, scale, nsplit,   \
                                (cudaStream_t) stream);
    switch (lat / 32) {
      TB_LAT_CASE(1) TB_LAT_CASE(2) TB_LAT_CASE(3) TB_LAT_CASE(4) TB_LAT_CASE(5) TB_LAT_CASE(6) TB_LAT_CASE(8) TB_LAT_CASE(12)
      TB_LAT_CASE(16)
      default: break;
    }
#undef TB_LAT_CASE
  }
  const int D = lat + rot_dim;
  const size_t smem = sizeof(float) * ((size_t) kKeyTile * (D + 1) + (size_t) kAttnWarps * (D + lat));
  if (smem > 227 * 1024) return -2;
  cudaStream_t s = (cudaStream_t) stream;
  dim3 grid(rows, (heads + kAttnWarps - 1) / kAttnWarps);
  static size_t raised_f = 48 * 1024, raised_b = 48 * 1024;
  if (dtype == TB_DT_F32) {
    if (smem > raised_f) {
      TB_CHECK_CUDA(cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
      raised_f = smem;
    }
    latent_attention_kernel<float><<<grid, kAttnWarps * 32, smem, s>>>((float*) out, (const float*) qa, (const float*) pool,
                                                                       tok_seq, tok_pos, block_table, max_blocks, page, heads,
                                                                       lat, rot_dim, scale);
  } else {
    if (smem > raised_b) {
      TB_CHECK_CUDA(cudaFuncSetAttribute(latent_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int) smem));
      raised_b = smem;
    }
    latent_attention_kernel<__nv_bfloat16><<<grid, kAttnWarps * 32, smem, s>>>(
        (__nv_bfloat16*) out, (const __nv_bfloat16*) qa, (const __nv_bfloat16*) pool, tok_seq, tok_pos, block_table,
        max_blocks, page, heads, lat, rot_dim, scale);
  }
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
