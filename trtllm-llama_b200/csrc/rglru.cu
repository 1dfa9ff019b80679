// Recurrent mixer kernels for a ragged in-flight batch: a per-channel causal convolution whose last taps - 1 inputs are
// carried per sequence, and the real-gated linear recurrence
//     S_t = a_t * S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t,   a_t = exp(-c * r_t * softplus(lam))
// whose state is carried per sequence in fp32.  Sequences own a slot of the state buffers; a sequence that stands at
// position 0 reads zeros whatever its slot held before, so a slot can be handed on without being cleared.
// Everything here is fp32 except the stored output of the recurrence, which is multiplied by the gate branch and
// rounded to the model's storage type for the projection that follows.
#include <cuda_bf16.h>

#include "common.cuh"
#include "../../include/trtllm_b200_ragged.h"

namespace tb {
namespace {

constexpr int kMaxTaps = 16;

__device__ __forceinline__ float ld_w(const void* p, int dtype, int64_t i) {
  return dtype == TB_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// one thread per (row, channel); channels fastest
__global__ void causal_conv1d_kernel(float* out, const float* x, const void* w, const void* bias, int w_dtype,
                                     const float* state, const int* tok_seq, const int* tok_pos, const int* seq_start,
                                     const int* seq_past, const int* seq_slot, int rows, int channels, int taps) {
  const int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x;
  if (i >= (int64_t) rows * channels) return;
  const int row = (int) (i / channels), ch = (int) (i % channels);
  const int e = tok_seq[row], pos = tok_pos[row], past = seq_past[e], start = seq_start[e];
  const float* st = state + (int64_t) seq_slot[e] * (taps - 1) * channels;
  float acc = bias ? ld_w(bias, w_dtype, ch) : 0.f;
  for (int k = 0; k < taps; ++k) {
    const int p = pos - (taps - 1 - k);              // absolute position of the input under tap k
    float v = 0.f;
    if (p >= past) v = x[(int64_t) (start + (p - past)) * channels + ch];
    else if (p >= 0) v = st[(int64_t) (taps - 1 - (past - p)) * channels + ch];   // state row j holds position past - (taps-1) + j
    acc = fmaf(ld_w(w, w_dtype, (int64_t) ch * taps + k), v, acc);
  }
  out[i] = acc;
}

// one thread per (sequence, channel): reads every old value it needs before it writes
__global__ void causal_conv1d_update_kernel(float* state, const float* x, int64_t ldx, const int* seq_start, const int* seq_len,
                                            const int* seq_past, const int* seq_slot, int seqs, int channels, int taps,
                                            int skip_single) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= seqs * channels) return;
  const int e = i / channels, ch = i % channels;
  const int len = seq_len[e], past = seq_past[e], start = seq_start[e];
  if (skip_single && len == 1) return;               // the convolution kernel moved this sequence's inputs on itself
  float* st = state + (int64_t) seq_slot[e] * (taps - 1) * channels;
  float keep[kMaxTaps];
  const int n = taps - 1;
  for (int j = 0; j < n; ++j) {
    const int p = past + len - n + j;                // absolute position the new state row j holds
    float v = 0.f;
    if (p >= past) v = x[(int64_t) (start + (p - past)) * ldx + ch];
    else if (p >= 0) v = st[(int64_t) (n - (past - p)) * channels + ch];
    keep[j] = v;
  }
  for (int j = 0; j < n; ++j) st[(int64_t) j * channels + ch] = keep[j];
}

template <typename T>
__global__ void rglru_scan_kernel(T* out, const float* u, const float* gates, const void* lam, int w_dtype, const T* y,
                                  float* state, const int* seq_start, const int* seq_len, const int* seq_past,
                                  const int* seq_slot, int seqs, int channels, int blocks, float c) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= seqs * channels) return;
  const int e = i / channels, ch = i % channels;
  const int bw = channels / blocks, b = ch / bw, j = ch % bw;
  const int len = seq_len[e], start = seq_start[e];
  float* sp = state + (int64_t) seq_slot[e] * channels + ch;
  float S = seq_past[e] > 0 ? *sp : 0.f;
  const float lm = ld_w(lam, w_dtype, ch);
  const float sp_lam = lm > 20.f ? lm : log1pf(expf(lm));
  const int64_t g_r = (int64_t) (b * 2) * bw + j, g_i = g_r + bw;
  for (int t = 0; t < len; ++t) {
    const int64_t row = start + t;
    const float r = 1.f / (1.f + expf(-gates[row * 2 * channels + g_r]));
    const float ig = 1.f / (1.f + expf(-gates[row * 2 * channels + g_i]));
    const float la = -c * r * sp_lam;
    const float a = expf(la);
    const float mult = sqrtf(-expm1f(2.f * la));
    S = fmaf(a, S, mult * ig * u[row * channels + ch]);
    float yv;
    if constexpr (sizeof(T) == 4) yv = y[row * channels + ch]; else yv = __bfloat162float(y[row * channels + ch]);
    const float o = S * yv;
    if constexpr (sizeof(T) == 4) out[row * channels + ch] = o; else out[row * channels + ch] = __float2bfloat16_rn(o);
  }
  *sp = S;
}


// Chunked form for long portions (prefill): the recurrence S_t = a_t S_(t-1) + b_t composes, so a sequence's rows are cut
// into chunks of kScanChunk rows; (1) every (chunk, channel) scans its rows from zero and keeps the product of its a's and its
// final value, (2) one thread per (sequence, channel) walks the chunk summaries in order, leaves every chunk's incoming
// state and the sequence's new state, (3) every (chunk, channel) scans again from its incoming state and writes S * y.
// Gates are recomputed in (3) instead of stored: two transcendental passes cost less than 16 bytes per element of traffic.
constexpr int kScanChunk = 32;

struct GateCoef { float a, b; };
__device__ __forceinline__ GateCoef rglru_coef(float gr, float gi, float uv, float c_sp) {
  const float r = 1.f / (1.f + expf(-gr));
  const float ig = 1.f / (1.f + expf(-gi));
  const float la = -c_sp * r;
  GateCoef k;
  k.a = expf(la);
  k.b = sqrtf(-expm1f(2.f * la)) * ig * uv;
  return k;
}

// grid (ceil(C / 128), max_chunks, seqs)
template <typename T, int PHASE>
__global__ void __launch_bounds__(128) rglru_chunk_kernel(T* out, const float* u, const float* gates, const void* lam, int w_dtype,
                                                          const T* y, float* ws, const int* seq_start, const int* seq_len,
                                                          int channels, int blocks, float c, int max_chunks) {
  const int ch = blockIdx.x * 128 + threadIdx.x, chunk = blockIdx.y, e = blockIdx.z;
  if (ch >= channels) return;
  const int len = seq_len[e], r0 = chunk * kScanChunk;
  if (r0 >= len) return;
  const int r1 = min(len, r0 + kScanChunk);
  const int bw = channels / blocks, b = ch / bw, j = ch % bw;
  const float lm = ld_w(lam, w_dtype, ch);
  const float c_sp = c * (lm > 20.f ? lm : log1pf(expf(lm)));
  const int64_t g_r = (int64_t) (b * 2) * bw + j, g_i = g_r + bw;
  const int64_t slot = ((int64_t) e * max_chunks + chunk) * channels + ch, plane = (int64_t) gridDim.z * max_chunks * channels;
  float S = PHASE == 1 ? 0.f : ws[2 * plane + slot], P = 1.f;
#pragma unroll 4
  for (int64_t row = seq_start[e] + r0; row < seq_start[e] + r1; ++row) {
    const GateCoef k = rglru_coef(gates[row * 2 * channels + g_r], gates[row * 2 * channels + g_i], u[row * channels + ch], c_sp);
    S = fmaf(k.a, S, k.b);
    if (PHASE == 1) {
      P *= k.a;
    } else {
      float yv;
      if constexpr (sizeof(T) == 4) yv = y[row * channels + ch]; else yv = __bfloat162float(y[row * channels + ch]);
      if constexpr (sizeof(T) == 4) out[row * channels + ch] = S * yv; else out[row * channels + ch] = __float2bfloat16_rn(S * yv);
    }
  }
  if (PHASE == 1) { ws[slot] = P; ws[plane + slot] = S; }
}

// one thread per (sequence, channel): carry the state through the chunk summaries
__global__ void rglru_carry_kernel(float* ws, float* state, const int* seq_len, const int* seq_past, const int* seq_slot, int seqs,
                                   int channels, int max_chunks) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= seqs * channels) return;
  const int e = i / channels, ch = i % channels;
  const int chunks = (seq_len[e] + kScanChunk - 1) / kScanChunk;
  const int64_t plane = (int64_t) seqs * max_chunks * channels;
  float* sp = state + (int64_t) seq_slot[e] * channels + ch;
  float S = seq_past[e] > 0 ? *sp : 0.f;
  for (int k = 0; k < chunks; ++k) {
    const int64_t slot = ((int64_t) e * max_chunks + k) * channels + ch;
    ws[2 * plane + slot] = S;
    S = fmaf(ws[slot], S, ws[plane + slot]);
  }
  *sp = S;
}

}  // namespace
}  // namespace tb

using namespace tb;

extern "C" int tb_causal_conv1d(float* out, const float* x, const void* w, const void* bias, int w_dtype, const float* state,
                                const int* tok_seq, const int* tok_pos, const int* seq_start, const int* seq_past,
                                const int* seq_slot, int rows, int channels, int taps, tb_stream_t stream) {
  if (!out || !x || !w || !state || !tok_seq || !tok_pos || !seq_start || !seq_past || !seq_slot || channels <= 0 ||
      taps < 1 || taps > kMaxTaps || rows < 0 || (w_dtype != TB_DT_F32 && w_dtype != TB_DT_BF16))
    return -1;
  if (rows == 0) return 0;
  const int64_t n = (int64_t) rows * channels;
  causal_conv1d_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, (cudaStream_t) stream>>>(
      out, x, w, bias, w_dtype, state, tok_seq, tok_pos, seq_start, seq_past, seq_slot, rows, channels, taps);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_causal_conv1d_update(float* state, const float* x, int64_t ldx, const int* seq_start, const int* seq_len,
                                       const int* seq_past, const int* seq_slot, int seqs, int channels, int taps,
                                       int skip_single, tb_stream_t stream) {
  if (!state || !x || !seq_start || !seq_len || !seq_past || !seq_slot || channels <= 0 || taps < 1 || taps > kMaxTaps ||
      seqs < 0)
    return -1;
  if (seqs == 0 || taps == 1) return 0;
  const int n = seqs * channels;
  causal_conv1d_update_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t) stream>>>(state, x, ldx, seq_start, seq_len, seq_past,
                                                                                   seq_slot, seqs, channels, taps, skip_single);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_rglru_scan(void* out, int dtype, const float* u, const float* gates, const void* lam, int w_dtype,
                             const void* y, float* state, const int* seq_start, const int* seq_len, const int* seq_past,
                             const int* seq_slot, int seqs, int channels, int blocks, float c, int max_len, float* workspace,
                             tb_stream_t stream) {
  if (!out || !u || !gates || !lam || !y || !state || !seq_start || !seq_len || !seq_past || !seq_slot || channels <= 0 ||
      blocks <= 0 || channels % blocks || seqs < 0)
    return -1;
  if ((dtype != TB_DT_F32 && dtype != TB_DT_BF16) || (w_dtype != TB_DT_F32 && w_dtype != TB_DT_BF16)) return -1;
  if (seqs == 0) return 0;
  const int n = seqs * channels;
  cudaStream_t s = (cudaStream_t) stream;
  if (workspace && max_len > kScanChunk && seqs <= 65535) {
    const int max_chunks = (max_len + kScanChunk - 1) / kScanChunk;
    if (max_chunks > 65535) return -2;
    dim3 grid((channels + 127) / 128, max_chunks, seqs);
    if (dtype == TB_DT_F32) {
      rglru_chunk_kernel<float, 1><<<grid, 128, 0, s>>>((float*) out, u, gates, lam, w_dtype, (const float*) y, workspace,
                                                        seq_start, seq_len, channels, blocks, c, max_chunks);
      rglru_carry_kernel<<<(n + 127) / 128, 128, 0, s>>>(workspace, state, seq_len, seq_past, seq_slot, seqs, channels, max_chunks);
      rglru_chunk_kernel<float, 2><<<grid, 128, 0, s>>>((float*) out, u, gates, lam, w_dtype, (const float*) y, workspace,
                                                        seq_start, seq_len, channels, blocks, c, max_chunks);
    } else {
      rglru_chunk_kernel<__nv_bfloat16, 1><<<grid, 128, 0, s>>>((__nv_bfloat16*) out, u, gates, lam, w_dtype,
                                                                (const __nv_bfloat16*) y, workspace, seq_start, seq_len,
                                                                channels, blocks, c, max_chunks);
      rglru_carry_kernel<<<(n + 127) / 128, 128, 0, s>>>(workspace, state, seq_len, seq_past, seq_slot, seqs, channels, max_chunks);
      rglru_chunk_kernel<__nv_bfloat16, 2><<<grid, 128, 0, s>>>((__nv_bfloat16*) out, u, gates, lam, w_dtype,
                                                                (const __nv_bfloat16*) y, workspace, seq_start, seq_len,
                                                                channels, blocks, c, max_chunks);
    }
    TB_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  if (dtype == TB_DT_F32)
    rglru_scan_kernel<float><<<(n + 63) / 64, 64, 0, s>>>((float*) out, u, gates, lam, w_dtype, (const float*) y, state,
                                                          seq_start, seq_len, seq_past, seq_slot, seqs, channels, blocks, c);
  else
    rglru_scan_kernel<__nv_bfloat16><<<(n + 63) / 64, 64, 0, s>>>((__nv_bfloat16*) out, u, gates, lam, w_dtype,
                                                                  (const __nv_bfloat16*) y, state, seq_start, seq_len,
                                                                  seq_past, seq_slot, seqs, channels, blocks, c);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
