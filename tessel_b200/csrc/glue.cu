// The memory-bound glue kernels of a decoder step: embedding gather, RMSNorm,
// rotary embedding of the queries, rotary + paged KV-cache write (also as one
// launch, rope_kv), the final norm of selected rows, and (beyond the
// reference) residual add, row argmax (whole rows, or a vocabulary split
// across ranks) and the device-side step advance. All are 16-byte vectorised; none needs shared-memory staging beyond
// a block reduction.
//
// Rounding follows tessel's interpreter: every f32 product, sum and quotient
// is rounded on its own (no fused multiply-add), so that the KV pages written
// here are bit-identical to the reference's CPU path for identical inputs.
#include <climits>
#include <cuda_fp8.h>

#include "common.cuh"

namespace tb {

namespace {

union H8 {
  uint4 u;
  __half h[8];
};

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;
}

// kernels/llm.tl:10-16. One block per token; a token outside [0, V) reads zeros.
__global__ void embed_kernel(const int* __restrict__ tok, const __half* __restrict__ E, float* __restrict__ X, int V,
                             int Dm) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int row = tok[t];
  const bool in = row >= 0 && row < V;
  const __half* e = E + (size_t)(in ? row : 0) * Dm;
  float* x = X + (size_t)t * Dm;
  if ((Dm & 7) == 0) {
    for (int c = threadIdx.x * 8; c < Dm; c += blockDim.x * 8) {
      H8 v;
      v.u = in ? *reinterpret_cast<const uint4*>(e + c) : make_uint4(0, 0, 0, 0);
      float4 a, b;
      a.x = __half2float(v.h[0]); a.y = __half2float(v.h[1]); a.z = __half2float(v.h[2]); a.w = __half2float(v.h[3]);
      b.x = __half2float(v.h[4]); b.y = __half2float(v.h[5]); b.z = __half2float(v.h[6]); b.w = __half2float(v.h[7]);
      *reinterpret_cast<float4*>(x + c) = a;
      *reinterpret_cast<float4*>(x + c + 4) = b;
    }
  } else {
    for (int c = threadIdx.x; c < Dm; c += blockDim.x) x[c] = in ? __half2float(e[c]) : 0.0f;
  }
}

// kernels/llm.tl:19-25 and :175-182 (idx != null gathers rows). One block per
// output row. The row is read once into registers when it fits (Dm <= 8192).
template <int PER>  // float4 chunks per thread
__global__ void rmsnorm_kernel(const float* __restrict__ X, const int* __restrict__ idx, const __half* __restrict__ W,
                               __half* __restrict__ Y, float eps, int T, int Dm) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const int b = blockIdx.x;
  int r = idx ? idx[b] : b;
  const bool in = r >= 0 && r < T;
  const float* x = X + (size_t)(in ? r : 0) * Dm;
  float4 v[PER];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 4;
    v[i] = (in && c < Dm) ? *reinterpret_cast<const float4*>(x + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += __fmul_rn(v[i].x, v[i].x);
    ss += __fmul_rn(v[i].y, v[i].y);
    ss += __fmul_rn(v[i].z, v[i].z);
    ss += __fmul_rn(v[i].w, v[i].w);
  }
  const float sum = block_sum(ss, red);
  const float ms = __fdiv_rn(sum, (float)Dm);
  const float rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 4;
    if (c < Dm) {
      const __half2 w01 = *reinterpret_cast<const __half2*>(W + c);
      const __half2 w23 = *reinterpret_cast<const __half2*>(W + c + 2);
      const float y0 = __fmul_rn(__fmul_rn(v[i].x, rs), __low2float(w01));
      const float y1 = __fmul_rn(__fmul_rn(v[i].y, rs), __high2float(w01));
      const float y2 = __fmul_rn(__fmul_rn(v[i].z, rs), __low2float(w23));
      const float y3 = __fmul_rn(__fmul_rn(v[i].w, rs), __high2float(w23));
      uint2 o;
      o.x = pack_h2(y0, y1);
      o.y = pack_h2(y2, y3);
      *reinterpret_cast<uint2*>(Y + (size_t)b * Dm + c) = o;
    }
  }
}

// Any Dm (two passes over the row).
__global__ void rmsnorm_generic_kernel(const float* __restrict__ X, const int* __restrict__ idx,
                                       const __half* __restrict__ W, __half* __restrict__ Y, float eps, int T, int Dm) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const int b = blockIdx.x;
  int r = idx ? idx[b] : b;
  const bool in = r >= 0 && r < T;
  const float* x = X + (size_t)(in ? r : 0) * Dm;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < Dm; c += blockDim.x) {
    const float v = in ? x[c] : 0.0f;
    ss += __fmul_rn(v, v);
  }
  const float sum = block_sum(ss, red);
  const float ms = __fdiv_rn(sum, (float)Dm);
  const float rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
  for (int c = threadIdx.x; c < Dm; c += blockDim.x) {
    const float v = in ? x[c] : 0.0f;
    Y[(size_t)b * Dm + c] = __float2half_rn(__fmul_rn(__fmul_rn(v, rs), __half2float(W[c])));
  }
}

// ---- FP8 mode (no counterpart in the reference: a separate, non-parity mode) -------------------
// A row of activations as E4M3 bytes and one f32 scale: scale = max|row| / 448 (1 for a zero
// row), byte = e4m3(x / scale) rounded to nearest even and saturated, the same arithmetic as the
// host's quantiser of the weights (tessel_b200/fp8.py), so both sides of a product are
// quantised by one rule.
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  __syncthreads();
  return t;
}

__device__ __forceinline__ unsigned char to_e4m3(float x) {
  return (unsigned char)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// quant_rows: X f16 [M, K] -> Q u8 [M, K], S f32 [M]. One block per row; K % 8 == 0.
__global__ void quant_rows_kernel(const __half* __restrict__ X, unsigned char* __restrict__ Q, float* __restrict__ S,
                                  int K) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const __half* x = X + (size_t)blockIdx.x * K;
  float mx = 0.f;
  for (int c = threadIdx.x * 8; c < K; c += blockDim.x * 8) {
    H8 v;
    v.u = *reinterpret_cast<const uint4*>(x + c);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(__half2float(v.h[j])));
  }
  mx = block_max(mx, red);
  const float scale = mx > 0.f ? __fdiv_rn(mx, 448.0f) : 1.0f;
  if (threadIdx.x == 0) S[blockIdx.x] = scale;
  unsigned char* q = Q + (size_t)blockIdx.x * K;
  for (int c = threadIdx.x * 8; c < K; c += blockDim.x * 8) {
    H8 v;
    v.u = *reinterpret_cast<const uint4*>(x + c);
    unsigned char b[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) b[j] = to_e4m3(__fdiv_rn(__half2float(v.h[j]), scale));
    *reinterpret_cast<uint2*>(q + c) = *reinterpret_cast<const uint2*>(b);
  }
}

// rmsnorm_q8: the RMSNorm of kernels/llm.tl:19-25 (y rounded to f16, as the reference's h is)
// followed by quant_rows of y, in one pass: X f32 [T, Dm], W f16 [Dm] -> Q u8 [T, Dm], S f32 [T].
template <int PER>  // float4 chunks per thread
__global__ void rmsnorm_q8_kernel(const float* __restrict__ X, const __half* __restrict__ W,
                                  unsigned char* __restrict__ Q, float* __restrict__ S, float eps, int Dm) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const int b = blockIdx.x;
  const float* x = X + (size_t)b * Dm;
  float4 v[PER];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 4;
    v[i] = c < Dm ? *reinterpret_cast<const float4*>(x + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += __fmul_rn(v[i].x, v[i].x);
    ss += __fmul_rn(v[i].y, v[i].y);
    ss += __fmul_rn(v[i].z, v[i].z);
    ss += __fmul_rn(v[i].w, v[i].w);
  }
  const float sum = block_sum(ss, red);
  const float ms = __fdiv_rn(sum, (float)Dm);
  const float rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
  float mx = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 4;
    if (c < Dm) {
      const __half2 w01 = *reinterpret_cast<const __half2*>(W + c);
      const __half2 w23 = *reinterpret_cast<const __half2*>(W + c + 2);
      // y as the f16 the unquantised path would have stored
      v[i].x = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(v[i].x, rs), __low2float(w01))));
      v[i].y = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(v[i].y, rs), __high2float(w01))));
      v[i].z = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(v[i].z, rs), __low2float(w23))));
      v[i].w = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(v[i].w, rs), __high2float(w23))));
      mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[i].x), fabsf(v[i].y))), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
    }
  }
  mx = block_max(mx, red);
  const float scale = mx > 0.f ? __fdiv_rn(mx, 448.0f) : 1.0f;
  if (threadIdx.x == 0) S[b] = scale;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 4;
    if (c < Dm) {
      uchar4 o;
      o.x = to_e4m3(__fdiv_rn(v[i].x, scale));
      o.y = to_e4m3(__fdiv_rn(v[i].y, scale));
      o.z = to_e4m3(__fdiv_rn(v[i].z, scale));
      o.w = to_e4m3(__fdiv_rn(v[i].w, scale));
      *reinterpret_cast<uchar4*>(Q + (size_t)b * Dm + c) = o;
    }
  }
}

// One rotated pair (kernels/llm.tl:85-88): products and sums rounded separately.
__device__ __forceinline__ void rotate(float x1, float x2, float c, float s, float& y1, float& y2) {
  y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
  y2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
}

// Rotates 8 pairs: x1/x2 are the 8 first-half / second-half values, at column i0 of the tables.
__device__ __forceinline__ void rotate8(const H8& x1, const H8& x2, const float* __restrict__ Cp,
                                        const float* __restrict__ Sp, bool in, H8& y1, H8& y2) {
  float c[8], s[8];
  if (in) {
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(Cp);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(Cp + 4);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(Sp);
    *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(Sp + 4);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) c[j] = s[j] = 0.0f;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float a, b;
    rotate(__half2float(x1.h[j]), __half2float(x2.h[j]), c[j], s[j], a, b);
    y1.h[j] = __float2half_rn(a);
    y2.h[j] = __float2half_rn(b);
  }
}

// kernels/llm.tl:78-88. Thread = 8 pairs of one (token, head). D % 16 == 0.
__global__ void rope_q_kernel(const __half* __restrict__ QKV, const int* __restrict__ pos, const float* __restrict__ Ct,
                              const float* __restrict__ St, __half* __restrict__ Q, int T, int W, int NPOS, int H,
                              int D) {
  pdl_launch();
  pdl_wait();
  const int d2 = D >> 1, per = d2 >> 3;  // 8-pair chunks per head
  const long long n = (long long)T * H * per;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % per);
    const int h = (int)((i / per) % H);
    const int t = (int)(i / ((long long)per * H));
    const int p = pos[t];
    const bool in = p >= 0 && p < NPOS;
    const __half* src = QKV + (size_t)t * W + h * D + ch * 8;
    H8 x1, x2, y1, y2;
    x1.u = *reinterpret_cast<const uint4*>(src);
    x2.u = *reinterpret_cast<const uint4*>(src + d2);
    const size_t to = (size_t)(in ? p : 0) * d2 + ch * 8;
    rotate8(x1, x2, Ct + to, St + to, in, y1, y2);
    __half* dst = Q + ((size_t)t * H + h) * D + ch * 8;
    *reinterpret_cast<uint4*>(dst) = y1.u;
    *reinterpret_cast<uint4*>(dst + d2) = y2.u;
  }
}

// kernels/llm.tl:93-112. Thread = 8 pairs of K and the matching 16 values of
// V of one (token, kv head). A slot outside [0, NS) drops the cache write
// (padding rows use slot == NS); the dense K, V rows are always written.
__global__ void kv_write_kernel(const __half* __restrict__ QKV, const int* __restrict__ pos,
                                const int* __restrict__ slot, const float* __restrict__ Ct,
                                const float* __restrict__ St, __half* __restrict__ Kc, __half* __restrict__ Vc,
                                __half* __restrict__ Kd, __half* __restrict__ Vd, int T, int W, int NPOS, int NS, int G,
                                int D) {
  pdl_launch();
  pdl_wait();
  const int d2 = D >> 1, per = d2 >> 3;
  const long long n = (long long)T * G * per;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % per);
    const int g = (int)((i / per) % G);
    const int t = (int)(i / ((long long)per * G));
    const int p = pos[t], at = slot[t];
    const bool in = p >= 0 && p < NPOS, keep = at >= 0 && at < NS;
    const int k0 = W - 2 * G * D + g * D;
    const __half* src = QKV + (size_t)t * W + k0 + ch * 8;
    H8 x1, x2, y1, y2;
    x1.u = *reinterpret_cast<const uint4*>(src);
    x2.u = *reinterpret_cast<const uint4*>(src + d2);
    const uint4 v1 = *reinterpret_cast<const uint4*>(src + G * D);
    const uint4 v2 = *reinterpret_cast<const uint4*>(src + G * D + d2);
    const size_t to = (size_t)(in ? p : 0) * d2 + ch * 8;
    rotate8(x1, x2, Ct + to, St + to, in, y1, y2);
    const size_t dd = ((size_t)t * G + g) * D + ch * 8;
    *reinterpret_cast<uint4*>(Kd + dd) = y1.u;
    *reinterpret_cast<uint4*>(Kd + dd + d2) = y2.u;
    *reinterpret_cast<uint4*>(Vd + dd) = v1;
    *reinterpret_cast<uint4*>(Vd + dd + d2) = v2;
    if (keep) {
      const size_t cd = ((size_t)at * G + g) * D + ch * 8;
      *reinterpret_cast<uint4*>(Kc + cd) = y1.u;
      *reinterpret_cast<uint4*>(Kc + cd + d2) = y2.u;
      *reinterpret_cast<uint4*>(Vc + cd) = v1;
      *reinterpret_cast<uint4*>(Vc + cd + d2) = v2;
    }
  }
}

// rope_q and kv_write in one launch (kernels/llm.tl:78-112): unit = 8 pairs of one (token, head),
// query heads first, then KV heads.
__global__ void rope_kv_kernel(const __half* __restrict__ QKV, const int* __restrict__ pos,
                               const int* __restrict__ slot, const float* __restrict__ Ct,
                               const float* __restrict__ St, __half* __restrict__ Q, __half* __restrict__ Kc,
                               __half* __restrict__ Vc, __half* __restrict__ Kd, __half* __restrict__ Vd, int T, int W,
                               int NPOS, int NS, int H, int G, int D) {
  pdl_launch();
  pdl_wait();
  const int d2 = D >> 1, per = d2 >> 3, HG = H + G;
  const long long n = (long long)T * HG * per;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % per);
    const int hh = (int)((i / per) % HG);
    const int t = (int)(i / ((long long)per * HG));
    const int p = pos[t];
    const bool in = p >= 0 && p < NPOS;
    const size_t to = (size_t)(in ? p : 0) * d2 + ch * 8;
    H8 x1, x2, y1, y2;
    if (hh < H) {
      const __half* src = QKV + (size_t)t * W + hh * D + ch * 8;
      x1.u = *reinterpret_cast<const uint4*>(src);
      x2.u = *reinterpret_cast<const uint4*>(src + d2);
      rotate8(x1, x2, Ct + to, St + to, in, y1, y2);
      __half* dst = Q + ((size_t)t * H + hh) * D + ch * 8;
      *reinterpret_cast<uint4*>(dst) = y1.u;
      *reinterpret_cast<uint4*>(dst + d2) = y2.u;
    } else {
      const int g = hh - H, at = slot[t];
      const bool keep = at >= 0 && at < NS;
      const __half* src = QKV + (size_t)t * W + (W - 2 * G * D + g * D) + ch * 8;
      x1.u = *reinterpret_cast<const uint4*>(src);
      x2.u = *reinterpret_cast<const uint4*>(src + d2);
      const uint4 v1 = *reinterpret_cast<const uint4*>(src + G * D);
      const uint4 v2 = *reinterpret_cast<const uint4*>(src + G * D + d2);
      rotate8(x1, x2, Ct + to, St + to, in, y1, y2);
      const size_t dd = ((size_t)t * G + g) * D + ch * 8;
      *reinterpret_cast<uint4*>(Kd + dd) = y1.u;
      *reinterpret_cast<uint4*>(Kd + dd + d2) = y2.u;
      *reinterpret_cast<uint4*>(Vd + dd) = v1;
      *reinterpret_cast<uint4*>(Vd + dd + d2) = v2;
      if (keep) {
        const size_t cd = ((size_t)at * G + g) * D + ch * 8;
        *reinterpret_cast<uint4*>(Kc + cd) = y1.u;
        *reinterpret_cast<uint4*>(Kc + cd + d2) = y2.u;
        *reinterpret_cast<uint4*>(Vc + cd) = v1;
        *reinterpret_cast<uint4*>(Vc + cd + d2) = v2;
      }
    }
  }
}

// R += P, f32, n % 4 == 0.
__global__ void residual_add_kernel(float* __restrict__ R, const float* __restrict__ P, long long n4) {
  pdl_launch();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 r = reinterpret_cast<float4*>(R)[i];
    const float4 p = reinterpret_cast<const float4*>(P)[i];
    r.x = __fadd_rn(r.x, p.x); r.y = __fadd_rn(r.y, p.y); r.z = __fadd_rn(r.z, p.z); r.w = __fadd_rn(r.w, p.w);
    reinterpret_cast<float4*>(R)[i] = r;
  }
}

// One rank's part of a row maximum over a vocabulary split across ranks: X holds columns
// [base, base + N) of the full row. Writes (value, global index as f32) to this rank's slot of
// pairs[R][M][2] and zeros to the other slots, so that a sum over ranks gathers every slot.
// The value is the first maximum among the columns that are not NaN; a slice with none gives
// (-inf, -1). Rank 0 reports (NaN, 0) when the row's very first value is NaN, because the
// sequential scan of src/llm/mod.rs:132-140 never leaves a NaN it starts on.
__global__ void argmax_partial_kernel(const float* __restrict__ X, float* __restrict__ pairs, int M, int N, int R,
                                      int rank, int base) {
  pdl_launch();
  pdl_wait();
  __shared__ float bv[32];
  __shared__ int bi[32];
  const int row = blockIdx.x;
  const float* x = X + (size_t)row * N;
  float best = -INFINITY;
  int at = INT_MAX;
  auto take = [&](float v, int c) {
    if (v > best || (v == best && c < at)) best = v, at = c;
  };
  if ((N & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    for (int c = threadIdx.x * 4; c < N; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(x + c);
      take(v.x, c), take(v.y, c + 1), take(v.z, c + 2), take(v.w, c + 3);
    }
  } else {
    for (int c = threadIdx.x; c < N; c += blockDim.x) take(x[c], c);
  }
  auto merge = [](float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, at, o);
    merge(best, at, ov, oi);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) {
    bv[w] = best;
    bi[w] = at;
  }
  __syncthreads();
  if (w == 0) {
    best = (l < nw) ? bv[l] : -INFINITY;
    at = (l < nw) ? bi[l] : INT_MAX;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, at, o);
      merge(best, at, ov, oi);
    }
    if (l < R) {
      float2 out = make_float2(0.f, 0.f);
      if (l == rank) {
        out = make_float2(best, at == INT_MAX ? -1.0f : (float)(base + at));
        if (base == 0 && x[0] != x[0]) out = make_float2(x[0], 0.f);
      }
      reinterpret_cast<float2*>(pairs)[(size_t)l * M + row] = out;
    }
  }
}

// The row maximum over the ranks' parts, taken in rank order so that the earliest index wins a
// tie; a NaN first value keeps index 0, as the sequential scan does.
__global__ void argmax_merge_kernel(const float* __restrict__ pairs, int* __restrict__ out, int M, int R) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  const float2* p = reinterpret_cast<const float2*>(pairs);
  float2 best = p[row];
  if (best.x == best.x) {
    for (int r = 1; r < R; ++r) {
      const float2 v = p[(size_t)r * M + row];
      if (v.y >= 0.f && (v.x > best.x || best.y < 0.f)) best = v;
    }
  }
  out[row] = best.y < 0.f ? 0 : (int)best.y;
}

// First index of each row's maximum (src/llm/mod.rs:132-140: a later equal
// value does not replace an earlier one; NaN never wins). One block per row.
__global__ void argmax_rows_kernel(const float* __restrict__ X, int* __restrict__ out, int N) {
  pdl_launch();
  pdl_wait();
  __shared__ float bv[32];
  __shared__ int bi[32];
  const float* x = X + (size_t)blockIdx.x * N;
  float best = x[0];
  int at = 0;
  // Thread-strided scan keeps, per thread, the earliest index of its maximum. A thread's
  // indices only grow, so a strict comparison already keeps the earliest.
  if ((N & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    for (int c = threadIdx.x * 4; c < N; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(x + c);
      if (v.x > best) best = v.x, at = c;
      if (v.y > best) best = v.y, at = c + 1;
      if (v.z > best) best = v.z, at = c + 2;
      if (v.w > best) best = v.w, at = c + 3;
    }
  } else {
    for (int c = threadIdx.x; c < N; c += blockDim.x) {
      const float v = x[c];
      if (v > best) best = v, at = c;
    }
  }
  auto merge = [](float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, at, o);
    merge(best, at, ov, oi);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) {
    bv[w] = best;
    bi[w] = at;
  }
  __syncthreads();
  if (w == 0) {
    best = (l < nw) ? bv[l] : x[0];
    at = (l < nw) ? bi[l] : 0;
    // x[0] with index 0 is a neutral element: it is in the row already.
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, at, o);
      merge(best, at, ov, oi);
    }
    if (l == 0) out[blockIdx.x] = at;
  }
}

// After a greedy decode step: row b < n takes its pick as the next token, moves one position
// on, and gets the cache slot of that position from its block table (page * P + offset, as
// src/llm/sched.rs:139-144 computes them on the host). Rows >= n stay padding. The picks are
// also appended to row `step` of the history hist[S, T].
__global__ void decode_advance_kernel(const int* __restrict__ picked, int* __restrict__ tok, int* __restrict__ pos,
                                      int* __restrict__ slot, int* __restrict__ lens, const int* __restrict__ table,
                                      int* __restrict__ hist, int MP, int n, int P) {
  pdl_launch();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n) return;
  const int p = pos[b] + 1;
  tok[b] = picked[b];
  hist[b] = picked[b];
  pos[b] = p;
  lens[b] = p + 1;
  const int col = p / P;
  slot[b] = col < MP ? table[(size_t)b * MP + col] * P + p % P : 0x7fffffff;  // past the table: dropped write
}

int grid_for(long long items, int block, int sms) {
  long long g = (items + block - 1) / block;
  const long long cap = (long long)sms * 16;
  if (g > cap) g = cap;
  return (int)(g < 1 ? 1 : g);
}

}  // namespace

int make_glue(Ctx* c, Op& op) {
  const auto& s = op.shapes;
  auto bad = [&](const char* why) { return fail(c, op.name + ": " + why); };
  switch (op.kind) {
    case K_EMBED:
      if (s[1].size() != 2 || s[2].size() != 2 || s[0][0] != s[2][0] || s[1][1] != s[2][1])
        return bad("shapes are tok[T], E[V,Dm], X[T,Dm]");
      break;
    case K_RMSNORM:
      if (s[0].size() != 2 || s[0] != s[2] || s[1][0] != s[0][1]) return bad("shapes are X[T,Dm], W[Dm], Y[T,Dm]");
      if (s[0][1] % 4) return bad("Dm must be a multiple of 4");
      break;
    case K_RMSNORM_ROWS:
      if (s[0].size() != 2 || s[3].size() != 2 || s[3][0] != s[1][0] || s[3][1] != s[0][1] || s[2][0] != s[0][1])
        return bad("shapes are X[T,Dm], idx[B], W[Dm], Y[B,Dm]");
      if (s[0][1] % 4) return bad("Dm must be a multiple of 4");
      break;
    case K_ROPE_Q: {
      if (s[4].size() != 3 || s[0].size() != 2 || s[2].size() != 2) return bad("shapes are QKV[T,W], pos[T], C, S, Q[T,H,D]");
      const int64_t D = s[4][2];
      if (D % 16 || s[2][1] != D / 2 || s[3] != s[2]) return bad("head_dim must be a multiple of 16, tables [NPOS, D/2]");
      if (s[0][1] % 8) return bad("W must be a multiple of 8");
      if (s[4][1] * D > s[0][1]) return bad("H*D exceeds W");
      break;
    }
    case K_KV_WRITE: {
      if (s[5].size() != 3 || s[7].size() != 3) return bad("caches are [NS,G,D], K and V [T,G,D]");
      const int64_t G = s[5][1], D = s[5][2];
      if (D % 16 || s[3][1] != D / 2) return bad("head_dim must be a multiple of 16, tables [NPOS, D/2]");
      if (s[0][1] % 8 || 2 * G * D > s[0][1]) return bad("W must be a multiple of 8 and hold 2*G*D columns");
      if (s[6] != s[5] || s[8] != s[7] || s[7][1] != G || s[7][2] != D) return bad("K/V shapes disagree");
      break;
    }
    case K_ROPE_KV: {
      // QKV[T,W], pos[T], slot[T], C, S [NPOS,D/2], Q[T,H,D], Kc, Vc [NS,G,D], K, V [T,G,D]
      if (s[0].size() != 2 || s[5].size() != 3 || s[6].size() != 3 || s[8].size() != 3 || s[3].size() != 2)
        return bad("shapes are QKV[T,W], pos[T], slot[T], C, S, Q[T,H,D], Kc, Vc[NS,G,D], K, V[T,G,D]");
      const int64_t H = s[5][1], D = s[5][2], G = s[6][1];
      if (D % 16 || s[3][1] != D / 2 || s[4] != s[3]) return bad("head_dim must be a multiple of 16, tables [NPOS, D/2]");
      if (s[0][1] % 8 || s[0][1] != (H + 2 * G) * D) return bad("W must be (H + 2G) * D");
      if (s[7] != s[6] || s[9] != s[8] || s[6][2] != D || s[8][1] != G || s[8][2] != D) return bad("K/V shapes disagree");
      break;
    }
    case K_RESIDUAL_ADD:
      if (s[0] != s[1]) return bad("R and P must have one shape");
      break;
    case K_ARGMAX_ROWS:
      if (s[0].size() != 2 || s[1][0] != s[0][0] || s[0][1] < 1) return bad("shapes are X[M,N], out[M]");
      break;
    case K_ARGMAX_PARTIAL:
      if (s[0].size() != 2 || s[1].size() != 3 || s[1][1] != s[0][0] || s[1][2] != 2 || s[0][1] < 1 || s[1][0] < 1 ||
          s[1][0] > 32)
        return bad("shapes are X[M,N], pairs[R,M,2] with 1 <= R <= 32");
      break;
    case K_ARGMAX_MERGE:
      if (s[0].size() != 3 || s[0][2] != 2 || s[1].size() != 1 || s[1][0] != s[0][1] || s[0][0] < 1)
        return bad("shapes are pairs[R,M,2], out[M]");
      break;
    case K_QUANT_ROWS:
      if (s[0].size() != 2 || s[1] != s[0] || s[2].size() != 1 || s[2][0] != s[0][0] || s[0][1] % 8)
        return bad("shapes are X[M,K], Q[M,K], S[M] with K a multiple of 8");
      break;
    case K_RMSNORM_Q8:
      if (s[0].size() != 2 || s[1].size() != 1 || s[1][0] != s[0][1] || s[2] != s[0] || s[3].size() != 1 ||
          s[3][0] != s[0][0] || s[0][1] % 4 || s[0][1] > 8192)
        return bad("shapes are X[T,Dm], W[Dm], Q[T,Dm], S[T] with Dm a multiple of 4, at most 8192");
      break;
    case K_DECODE_ADVANCE:
      if (s[5].size() != 2 || s[5][0] != s[0][0] || s[6].size() != 2 || s[6][1] != s[0][0])
        return bad("shapes are picked[T], tok[T], pos[T], slot[T], lens[T], table[T,MP], hist[S,T]");
      break;
    default:
      return bad("not a glue kernel");
  }
  return 0;
}

int launch_glue(Ctx* c, Op& op, const uint64_t* a) {
  const auto& s = op.shapes;
  switch (op.kind) {
    case K_EMBED: {
      const int T = (int)s[0][0], V = (int)s[1][0], Dm = (int)s[1][1];
      if (T == 0) return 0;
      TB_CUDA(c, launch_k(c, embed_kernel, dim3(T), dim3(128), 0, 1, (const int*)a[0], (const __half*)a[1], (float*)a[2], V, Dm));
      break;
    }
    case K_RMSNORM:
    case K_RMSNORM_ROWS: {
      const bool rows = op.kind == K_RMSNORM_ROWS;
      const int T = (int)s[0][0], Dm = (int)s[0][1];
      const int B = rows ? (int)s[1][0] : T;
      if (B == 0) return 0;
      const float* X = (const float*)a[0];
      const int* idx = rows ? (const int*)a[1] : nullptr;
      const __half* W = (const __half*)a[rows ? 2 : 1];
      __half* Y = (__half*)a[rows ? 3 : 2];
      const float eps = bits_f32(a[rows ? 4 : 3]);
      const int chunks = Dm / 4;
      if (chunks <= 256)
        TB_CUDA(c, launch_k(c, rmsnorm_kernel<1>, dim3(B), dim3(256), 0, 1, X, idx, W, Y, eps, T, Dm));
      else if (chunks <= 512)
        TB_CUDA(c, launch_k(c, rmsnorm_kernel<2>, dim3(B), dim3(256), 0, 1, X, idx, W, Y, eps, T, Dm));
      else if (chunks <= 1024)
        TB_CUDA(c, launch_k(c, rmsnorm_kernel<4>, dim3(B), dim3(256), 0, 1, X, idx, W, Y, eps, T, Dm));
      else if (chunks <= 2048)
        TB_CUDA(c, launch_k(c, rmsnorm_kernel<8>, dim3(B), dim3(256), 0, 1, X, idx, W, Y, eps, T, Dm));
      else
        TB_CUDA(c, launch_k(c, rmsnorm_generic_kernel, dim3(B), dim3(256), 0, 1, X, idx, W, Y, eps, T, Dm));
      break;
    }
    case K_ROPE_Q: {
      const int T = (int)s[0][0], W = (int)s[0][1], NPOS = (int)s[2][0], H = (int)s[4][1], D = (int)s[4][2];
      const long long n = (long long)T * H * (D / 16);
      if (n == 0) return 0;
      TB_CUDA(c, launch_k(c, rope_q_kernel, dim3(grid_for(n, 256, c->sm_count)), dim3(256), 0, 1, (const __half*)a[0], (const int*)a[1],
                                                                   (const float*)a[2], (const float*)a[3],
                                                                   (__half*)a[4], T, W, NPOS, H, D));
      break;
    }
    case K_KV_WRITE: {
      const int T = (int)s[0][0], W = (int)s[0][1], NPOS = (int)s[3][0], NS = (int)s[5][0], G = (int)s[5][1],
                D = (int)s[5][2];
      const long long n = (long long)T * G * (D / 16);
      if (n == 0) return 0;
      TB_CUDA(c, launch_k(c, kv_write_kernel, dim3(grid_for(n, 128, c->sm_count)), dim3(128), 0, 1, 
          (const __half*)a[0], (const int*)a[1], (const int*)a[2], (const float*)a[3], (const float*)a[4],
          (__half*)a[5], (__half*)a[6], (__half*)a[7], (__half*)a[8], T, W, NPOS, NS, G, D));
      break;
    }
    case K_ROPE_KV: {
      const int T = (int)s[0][0], W = (int)s[0][1], NPOS = (int)s[3][0], H = (int)s[5][1], D = (int)s[5][2],
                NS = (int)s[6][0], G = (int)s[6][1];
      const long long n = (long long)T * (H + G) * (D / 16);
      if (n == 0) return 0;
      TB_CUDA(c, launch_k(c, rope_kv_kernel, dim3(grid_for(n, 128, c->sm_count)), dim3(128), 0, 1, (const __half*)a[0],
                          (const int*)a[1], (const int*)a[2], (const float*)a[3], (const float*)a[4], (__half*)a[5],
                          (__half*)a[6], (__half*)a[7], (__half*)a[8], (__half*)a[9], T, W, NPOS, NS, H, G, D));
      break;
    }
    case K_RESIDUAL_ADD: {
      long long n = 1;
      for (int64_t d : s[0]) n *= d;
      if (n % 4) return fail(c, "residual_add: element count must be a multiple of 4");
      if (n == 0) return 0;
      TB_CUDA(c, launch_k(c, residual_add_kernel, dim3(grid_for(n / 4, 256, c->sm_count)), dim3(256), 0, 1, (float*)a[0], (const float*)a[1], n / 4));
      break;
    }
    case K_ARGMAX_ROWS: {
      const int M = (int)s[0][0], N = (int)s[0][1];
      if (M == 0) return 0;
      TB_CUDA(c, launch_k(c, argmax_rows_kernel, dim3(M), dim3(1024), 0, 1, (const float*)a[0], (int*)a[1], N));
      break;
    }
    case K_ARGMAX_PARTIAL: {
      const int M = (int)s[0][0], N = (int)s[0][1], R = (int)s[1][0];
      const int rank = (int)(uint32_t)a[2], base = (int)(uint32_t)a[3];
      if (rank < 0 || rank >= R || base < 0 || (long long)base + N > (1 << 24))
        return fail(c, "argmax_partial: 0 <= rank < R and base + N <= 2^24 (indices travel as f32)");
      if (M == 0) return 0;
      TB_CUDA(c, launch_k(c, argmax_partial_kernel, dim3(M), dim3(1024), 0, 1, (const float*)a[0], (float*)a[1], M, N, R, rank, base));
      break;
    }
    case K_ARGMAX_MERGE: {
      const int R = (int)s[0][0], M = (int)s[0][1];
      if (M == 0) return 0;
      TB_CUDA(c, launch_k(c, argmax_merge_kernel, dim3((M + 127) / 128), dim3(128), 0, 1, (const float*)a[0], (int*)a[1], M, R));
      break;
    }
    case K_QUANT_ROWS: {
      const int M = (int)s[0][0], K = (int)s[0][1];
      if (M == 0 || K == 0) return 0;
      TB_CUDA(c, launch_k(c, quant_rows_kernel, dim3(M), dim3(256), 0, 1, (const __half*)a[0], (unsigned char*)a[1],
                          (float*)a[2], K));
      break;
    }
    case K_RMSNORM_Q8: {
      const int T = (int)s[0][0], Dm = (int)s[0][1];
      if (T == 0) return 0;
      const float* X = (const float*)a[0];
      const __half* W = (const __half*)a[1];
      unsigned char* Q = (unsigned char*)a[2];
      float* S = (float*)a[3];
      const float eps = bits_f32(a[4]);
      const int chunks = Dm / 4;
      if (chunks <= 256)
        TB_CUDA(c, launch_k(c, rmsnorm_q8_kernel<1>, dim3(T), dim3(256), 0, 1, X, W, Q, S, eps, Dm));
      else if (chunks <= 512)
        TB_CUDA(c, launch_k(c, rmsnorm_q8_kernel<2>, dim3(T), dim3(256), 0, 1, X, W, Q, S, eps, Dm));
      else if (chunks <= 1024)
        TB_CUDA(c, launch_k(c, rmsnorm_q8_kernel<4>, dim3(T), dim3(256), 0, 1, X, W, Q, S, eps, Dm));
      else
        TB_CUDA(c, launch_k(c, rmsnorm_q8_kernel<8>, dim3(T), dim3(256), 0, 1, X, W, Q, S, eps, Dm));
      break;
    }
    case K_DECODE_ADVANCE: {
      const int T = (int)s[0][0], MP = (int)s[5][1];
      const int n = (int)(uint32_t)a[7], P = (int)(uint32_t)a[8], step = (int)(uint32_t)a[9];
      if (n < 0 || n > T || P < 1) return fail(c, "decode_advance: 0 <= n <= T and P >= 1");
      if (step < 0 || step >= (int)s[6][0]) return fail(c, "decode_advance: step outside the history");
      if (n == 0) return 0;
      TB_CUDA(c, launch_k(c, decode_advance_kernel, dim3((n + 127) / 128), dim3(128), 0, 1, (const int*)a[0], (int*)a[1], (int*)a[2], (int*)a[3],
                                                             (int*)a[4], (const int*)a[5], (int*)a[6] + (size_t)step * T,
                                                             MP, n, P));
      break;
    }
    default:
      return fail(c, op.name + ": not a glue kernel");
  }
  c->launches += 1;
  TB_CUDA(c, cudaGetLastError());
  return 0;
}

}  // namespace tb
