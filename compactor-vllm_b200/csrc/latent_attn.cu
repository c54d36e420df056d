// Latent attention: queries and keys/values go through low-rank latents; the cache holds, per token, ONE row
// [c | k_rot] of kv_rank + rot_dim numbers shared by all heads (c = the RMS-normed latent, k_rot = the rotated key
// part).  Attention runs in the latent space: with q_abs[h] = W_uk[h]^T q_plain[h] the score is
// (q_abs[h] . c + q_rot[h] . k_rot) * scale and the head's output is W_uv[h] (sum_j p_j c_j), i.e. attention with one
// key/value head of row size kv_rank + rot_dim whose values are the first kv_rank columns of its keys
// (cvllm_bias_attn_* with v_stride).  This file holds the steps around that attention and the library GEMMs:
//   cvllm_latent_norm_store   RMS norm of the query latent; RMS norm of the kv latent, rotation of the shared key
//                             part, both written to the token's cache row
//   cvllm_latent_q_rope       rotation of every head's rotated query part into the attention's query rows
//   cvllm_sigmoid_gate        x * sigmoid(gate), element by element
// Rotation ("rotate half"): element i of a part of R numbers pairs with element i + R/2; the pair (u, v) at position
// p becomes (u cos a - v sin a, v cos a + u sin a), a = p * inv_freq[i].  Angles and their sines are computed in
// 64-bit (inv_freq is a 64-bit table the caller fills with base ** (-2 i / R)), norms in 32-bit.
#include "common.cuh"

namespace cvllm {
namespace {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int kThreads = 128;

__device__ __forceinline__ float block_sum128(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

// cos / sin of position * inv_freq[i] for i < half, into shared memory (fp32 values of 64-bit angles)
__device__ __forceinline__ void fill_cos_sin(float* cs, float* sn, const double* __restrict__ inv_freq, int half,
                                             int pos) {
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double s, c;
    sincos((double)pos * inv_freq[i], &s, &c);
    cs[i] = (float)c;
    sn[i] = (float)s;
  }
}

// One CTA per token.  proj row: the query latent at q_off (q_rank numbers), the kv latent + shared key part at kv_off
// (kv_rank + R numbers; kv_off < 0: this layer has none of its own).
template <typename T>
__global__ void __launch_bounds__(kThreads) latent_norm_store_kernel(
    const T* __restrict__ proj, int64_t p_stride, int q_off, int q_rank, int kv_off, int kv_rank, int R,
    const float* __restrict__ q_w, const float* __restrict__ kv_w, float eps, const double* __restrict__ inv_freq,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_slot, T* __restrict__ cq_out,
    T* __restrict__ cache, const int32_t* __restrict__ table, int64_t table_stride_slot, int page_size,
    int32_t* __restrict__ lens, int reserved_slot) {
  extern __shared__ float sm[];     // cos[R/2], sin[R/2]
  __shared__ float red[4];
  const int t = blockIdx.x;
  const T* row = proj + (int64_t)t * p_stride;
  {
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += kThreads) {
      const float v = to_f<T>(row[q_off + i]);
      ss += v * v;
    }
    ss = block_sum128(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += kThreads)
      cq_out[(int64_t)t * q_rank + i] = from_f<T>(to_f<T>(row[q_off + i]) * inv * q_w[i]);
  }
  if (kv_off < 0) return;
  const int slot = token_slot[t];
  if (slot == reserved_slot) return;
  const int pos = positions[t];
  const int half = R / 2;
  float* cs = sm;
  float* sn = sm + half;
  fill_cos_sin(cs, sn, inv_freq, half, pos);
  const int lp = pos / page_size;
  const int page = table[(int64_t)slot * table_stride_slot + lp];
  T* dst = cache + ((int64_t)page * page_size + (pos - lp * page_size)) * (kv_rank + R);
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += kThreads) {
    const float v = to_f<T>(row[kv_off + i]);
    ss += v * v;
  }
  ss = block_sum128(ss, red);   // its barriers also publish cos / sin
  const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < kv_rank; i += kThreads)
    dst[i] = from_f<T>(to_f<T>(row[kv_off + i]) * inv * kv_w[i]);
  const T* kr = row + kv_off + kv_rank;
  for (int i = threadIdx.x; i < half; i += kThreads) {
    const float u = to_f<T>(kr[i]), v = to_f<T>(kr[i + half]);
    dst[kv_rank + i] = from_f<T>(u * cs[i] - v * sn[i]);
    dst[kv_rank + half + i] = from_f<T>(v * cs[i] + u * sn[i]);
  }
  if (threadIdx.x == 0 && lens) atomicMax(lens + slot, pos + 1);
}

// One CTA per token: q [T, H, D + R] -> q_full[t, h, off + 0 .. R) = rotate(q[t, h, D .. D + R)).
template <typename T>
__global__ void __launch_bounds__(kThreads) latent_q_rope_kernel(
    const T* __restrict__ q, int64_t q_stride, int H, int D, int R, const double* __restrict__ inv_freq,
    const int32_t* __restrict__ positions, T* __restrict__ q_full, int64_t f_stride, int f_head, int off) {
  extern __shared__ float sm[];
  const int t = blockIdx.x;
  const int half = R / 2;
  float* cs = sm;
  float* sn = sm + half;
  fill_cos_sin(cs, sn, inv_freq, half, positions[t]);
  __syncthreads();
  for (int i = threadIdx.x; i < H * half; i += kThreads) {
    const int h = i / half, j = i - h * half;
    const T* src = q + (int64_t)t * q_stride + (int64_t)h * (D + R) + D;
    T* dst = q_full + (int64_t)t * f_stride + (int64_t)h * f_head + off;
    const float u = to_f<T>(src[j]), v = to_f<T>(src[j + half]);
    dst[j] = from_f<T>(u * cs[j] - v * sn[j]);
    dst[j + half] = from_f<T>(v * cs[j] + u * sn[j]);
  }
}

template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ x, int64_t x_stride, const T* __restrict__ g,
                                    int64_t g_stride, T* __restrict__ out, int64_t o_stride, int64_t rows, int width) {
  const int64_t total = rows * (int64_t)width;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / width;
    const int c = (int)(i - t * width);
    const float gv = to_f<T>(g[t * g_stride + c]);
    out[t * o_stride + c] = from_f<T>(to_f<T>(x[t * x_stride + c]) / (1.0f + expf(-gv)));
  }
}

}  // namespace
}  // namespace cvllm

using namespace cvllm;

static int latent_dtype_ok(int dtype) { return dtype == CVLLM_BF16 || dtype == CVLLM_F32; }

extern "C" int cvllm_latent_norm_store(const void* proj, int64_t proj_stride, int q_off, int q_rank, int kv_off,
                                       int kv_rank, int rot_dim, const float* q_weight, const float* kv_weight,
                                       float eps, const double* inv_freq, const int32_t* positions,
                                       const int32_t* token_slot, void* cq_out, void* cache,
                                       const int32_t* page_table, int64_t table_stride_slot, int page_size,
                                       int32_t* lens, int T, int reserved_slot, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(T >= 0 && q_rank > 0 && q_off >= 0 && rot_dim >= 0 && rot_dim % 2 == 0);
  if (T == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(proj && q_weight && cq_out && latent_dtype_ok(dtype));
  if (kv_off >= 0)
    CVLLM_CHECK_ARG(kv_rank > 0 && kv_weight && positions && token_slot && cache && page_table && page_size > 0 &&
                    (rot_dim == 0 || inv_freq));
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)rot_dim * sizeof(float);
  CVLLM_CHECK_SUPPORTED(smem <= 48 * 1024);
  if (dtype == CVLLM_BF16)
    latent_norm_store_kernel<__nv_bfloat16><<<T, kThreads, smem, st>>>(
        static_cast<const __nv_bfloat16*>(proj), proj_stride, q_off, q_rank, kv_off, kv_rank, rot_dim, q_weight,
        kv_weight, eps, inv_freq, positions, token_slot, static_cast<__nv_bfloat16*>(cq_out),
        static_cast<__nv_bfloat16*>(cache), page_table, table_stride_slot, page_size, lens, reserved_slot);
  else
    latent_norm_store_kernel<float><<<T, kThreads, smem, st>>>(
        static_cast<const float*>(proj), proj_stride, q_off, q_rank, kv_off, kv_rank, rot_dim, q_weight, kv_weight, eps,
        inv_freq, positions, token_slot, static_cast<float*>(cq_out), static_cast<float*>(cache), page_table,
        table_stride_slot, page_size, lens, reserved_slot);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_latent_q_rope(const void* q, int64_t q_stride, int H, int D, int rot_dim, const double* inv_freq,
                                   const int32_t* positions, void* q_full, int64_t full_stride, int full_head, int off,
                                   int T, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(T >= 0 && H > 0 && D >= 0 && rot_dim >= 0 && rot_dim % 2 == 0 && off >= 0);
  if (T == 0 || rot_dim == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(q && inv_freq && positions && q_full && latent_dtype_ok(dtype) && off + rot_dim <= full_head);
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)rot_dim * sizeof(float);
  CVLLM_CHECK_SUPPORTED(smem <= 48 * 1024);
  if (dtype == CVLLM_BF16)
    latent_q_rope_kernel<__nv_bfloat16><<<T, kThreads, smem, st>>>(
        static_cast<const __nv_bfloat16*>(q), q_stride, H, D, rot_dim, inv_freq, positions,
        static_cast<__nv_bfloat16*>(q_full), full_stride, full_head, off);
  else
    latent_q_rope_kernel<float><<<T, kThreads, smem, st>>>(static_cast<const float*>(q), q_stride, H, D, rot_dim,
                                                           inv_freq, positions, static_cast<float*>(q_full),
                                                           full_stride, full_head, off);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_sigmoid_gate(const void* x, int64_t x_stride, const void* gate, int64_t g_stride, void* out,
                                  int64_t o_stride, int64_t rows, int width, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(rows >= 0 && width > 0);
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(x && gate && out && latent_dtype_ok(dtype));
  auto st = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * (int64_t)width;
  const int64_t want = (total + 255) / 256, cap = (int64_t)sm_count() * 16;
  const int grid = (int)(want < cap ? want : cap);
  if (dtype == CVLLM_BF16)
    sigmoid_gate_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), x_stride, static_cast<const __nv_bfloat16*>(gate), g_stride,
        static_cast<__nv_bfloat16*>(out), o_stride, rows, width);
  else
    sigmoid_gate_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), x_stride,
                                                     static_cast<const float*>(gate), g_stride,
                                                     static_cast<float*>(out), o_stride, rows, width);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}
