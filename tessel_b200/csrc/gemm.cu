// The projections of a decoder step on tcgen05 tensor cores:
//   linear           Y f16 = X W^T            kernels/llm.tl:28-36
//   linear_residual  R f32 += X W^T           kernels/llm.tl:39-47
//   logits           Y f32 = X W^T            kernels/llm.tl:50-58
//   gate_up          Y f16 = silu(X Wg^T) * (X Wu^T)   kernels/llm.tl:62-73
//   matmul           C f16 = A B, B [K,N] row-major    kernels/matmul.tl:3-17
//   linear_f32       Y f32 = X W^T (a tensor-parallel partial; no counterpart)
//
// One CTA computes a 128 x BN tile of the output. Warp 0 streams 64-wide K
// slices of both operands into a shared-memory ring with TMA (128-byte
// swizzle); one thread of warp 1 issues tcgen05.mma (M = 128, N = BN or 2 BN,
// K = 16, f16 in, f32 accumulate) into tensor memory and releases ring slots
// with tcgen05.commit; warps 2-5 read the finished accumulator out of tensor
// memory (one row per thread) and apply the epilogue. gate_up loads the Wg and
// Wu tiles side by side so that one MMA of N = 2 BN produces both products
// from one read of X. Rows beyond M and columns beyond N are zero-filled by
// TMA on the way in and masked on the way out.
//
// Shapes whose row pitch is not a multiple of 16 bytes (which TMA cannot
// address) take a plain tiled CUDA-core kernel with the same epilogues.
#include "common.cuh"

namespace tb {

namespace {

enum Epi : int { EPI_F16 = 0, EPI_RESID = 1, EPI_F32 = 2, EPI_GATE_UP = 3 };

constexpr int BM = 128, BK = 64;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  void* out;
  int M, N, K;
  unsigned int* status;
};

template <int BN, int EPI>
struct GemmCfg {
  static constexpr int NB = EPI == EPI_GATE_UP ? 2 * BN : BN;  // B rows per stage = MMA N
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = NB * BK * 2;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = (200 * 1024) / STAGE > 8 ? 8 : (200 * 1024) / STAGE;
  static constexpr int TMEM_COLS = NB <= 32 ? 32 : NB <= 64 ? 64 : NB <= 128 ? 128 : NB <= 256 ? 256 : 512;
  static constexpr int BAR_OFF = STAGES * STAGE;
  static constexpr int SMEM = BAR_OFF + (2 * STAGES + 1) * 8 + 16 + 1024;
  static_assert(NB % 16 == 0 && NB <= 256, "UMMA N");
};

__device__ __forceinline__ float silu_mul(float g, float u) {
  // g / (1 + exp(-g)) * u with each step rounded, as kernels/llm.tl:73 evaluates it.
  const float e = expf(-g);
  return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, e)), u);
}

// B_MN: B is a [K, N] row-major array (N-major operand); else W [N, K] (K-major).
template <int BN, int EPI, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                const __grid_constant__ CUtensorMap mapB2, const GemmParams p) {
  using Cfg = GemmCfg<BN, EPI>;
  constexpr int NB = Cfg::NB, STAGES = Cfg::STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + Cfg::BAR_OFF);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int nk = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      prefetch_tmap(&mapA);
      prefetch_tmap(&mapB);
      if (EPI == EPI_GATE_UP) prefetch_tmap(&mapB2);
      for (int i = 0; i < nk; ++i) {
        const int s = i % STAGES, k = i / STAGES;
        mbar_wait(&empty[s], (k & 1) ^ 1, p.status, 201);
        mbar_expect_tx(&full[s], Cfg::STAGE);
        unsigned char* a = smem + s * Cfg::STAGE;
        unsigned char* b = a + Cfg::A_BYTES;
        tma_load_2d(a, &mapA, &full[s], i * BK, m0);
        if (B_MN) {
          // 64-column blocks of [64 k-rows x 128 bytes] each.
#pragma unroll
          for (int nb = 0; nb < BN / 64; ++nb) tma_load_2d(b + nb * (BK * 128), &mapB, &full[s], n0 + nb * 64, i * BK);
        } else {
          tma_load_2d(b, &mapB, &full[s], i * BK, n0);
          if (EPI == EPI_GATE_UP) tma_load_2d(b + BN * BK * 2, &mapB2, &full[s], i * BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16(BM, NB, 0, B_MN ? 1 : 0);
      for (int i = 0; i < nk; ++i) {
        const int s = i % STAGES, k = i / STAGES;
        mbar_wait(&full[s], k & 1, p.status, 202);
        tc_fence_after();
        const uint32_t a = smem_u32(smem + s * Cfg::STAGE);
        const uint32_t b = a + Cfg::A_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(a + kk * 32, 16, 1024);
          const uint64_t bd = B_MN ? umma_desc_sw128(b + kk * 2048, BK * 128, 1024)
                                   : umma_desc_sw128(b + kk * 32, 16, 1024);
          umma_f16(tmem, ad, bd, idesc, (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);  // frees the slot once these MMAs have read it
      }
      umma_commit(acc_full);
    }
  } else {
    // ---- epilogue: 4 warps, TMEM lane quadrant = warp % 4 ------------------
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    mbar_wait(acc_full, 0, p.status, 203);
    tc_fence_after();
    const bool row_ok = row < p.M;
    const bool vec_ok = (p.N % 8) == 0;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + c0, r);
      uint32_t r2[32];
      if (EPI == EPI_GATE_UP) tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + BN + c0, r2);
      tmem_ld_wait();
      const int col = n0 + c0;
      if (!row_ok || col >= p.N) continue;
      const bool fullw = col + 32 <= p.N && vec_ok;
      if (EPI == EPI_F16 || EPI == EPI_GATE_UP) {
        __half* y = (__half*)p.out + (size_t)row * p.N + col;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          v[j] = EPI == EPI_GATE_UP ? silu_mul(__uint_as_float(r[j]), __uint_as_float(r2[j])) : __uint_as_float(r[j]);
        if (fullw) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_h2(v[j], v[j + 1]);
            o.y = pack_h2(v[j + 2], v[j + 3]);
            o.z = pack_h2(v[j + 4], v[j + 5]);
            o.w = pack_h2(v[j + 6], v[j + 7]);
            *reinterpret_cast<uint4*>(y + j) = o;
          }
        } else {
          for (int j = 0; j < 32 && col + j < p.N; ++j) y[j] = __float2half_rn(v[j]);
        }
      } else {
        float* y = (float*)p.out + (size_t)row * p.N + col;
        if (fullw) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 o = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                   __uint_as_float(r[j + 3]));
            if (EPI == EPI_RESID) {
              const float4 old = *reinterpret_cast<const float4*>(y + j);
              o.x = __fadd_rn(old.x, o.x);
              o.y = __fadd_rn(old.y, o.y);
              o.z = __fadd_rn(old.z, o.z);
              o.w = __fadd_rn(old.w, o.w);
            }
            *reinterpret_cast<float4*>(y + j) = o;
          }
        } else {
          for (int j = 0; j < 32 && col + j < p.N; ++j)
            y[j] = EPI == EPI_RESID ? __fadd_rn(y[j], __uint_as_float(r[j])) : __uint_as_float(r[j]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// CUDA-core path for pitches TMA cannot address: 32 x 32 output tile per block.
template <int EPI, bool B_MN>
__global__ void gemm_plain_kernel(const __half* __restrict__ A, const __half* __restrict__ B,
                                  const __half* __restrict__ B2, void* __restrict__ out, int M, int N, int K) {
  __shared__ float sa[32][33], sb[32][33], sb2[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
  const int m0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  float acc[4] = {0, 0, 0, 0}, acc2[4] = {0, 0, 0, 0};
  for (int k0 = 0; k0 < K; k0 += 32) {
    for (int r = ty; r < 32; r += 8) {
      const int m = m0 + r, k = k0 + tx, n = n0 + r;
      sa[r][tx] = (m < M && k < K) ? __half2float(A[(size_t)m * K + k]) : 0.f;
      if (B_MN) {
        // sb[k][n]
        const int kk = k0 + r, nn = n0 + tx;
        sb[r][tx] = (kk < K && nn < N) ? __half2float(B[(size_t)kk * N + nn]) : 0.f;
      } else {
        sb[r][tx] = (n < N && k < K) ? __half2float(B[(size_t)n * K + k]) : 0.f;  // sb[n][k]
        if (EPI == EPI_GATE_UP) sb2[r][tx] = (n < N && k < K) ? __half2float(B2[(size_t)n * K + k]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 8 * i;
      float s = acc[i], s2 = acc2[i];
      for (int k = 0; k < 32; ++k) {
        const float bv = B_MN ? sb[k][tx] : sb[tx][k];
        s = fmaf(sa[r][k], bv, s);
        if (EPI == EPI_GATE_UP) s2 = fmaf(sa[r][k], sb2[tx][k], s2);
      }
      acc[i] = s;
      acc2[i] = s2;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty + 8 * i, n = n0 + tx;
    if (m >= M || n >= N) continue;
    const size_t o = (size_t)m * N + n;
    if (EPI == EPI_F16)
      ((__half*)out)[o] = __float2half_rn(acc[i]);
    else if (EPI == EPI_GATE_UP)
      ((__half*)out)[o] = __float2half_rn(silu_mul(acc[i], acc2[i]));
    else if (EPI == EPI_RESID)
      ((float*)out)[o] = __fadd_rn(((float*)out)[o], acc[i]);
    else
      ((float*)out)[o] = acc[i];
  }
}

struct GemmShape {
  int M, N, K;
};

GemmShape gemm_shape(const Op& op) {
  const auto& s = op.shapes;
  GemmShape g;
  g.M = (int)s[0][0];
  g.K = (int)s[0][1];
  g.N = op.kind == K_MATMUL ? (int)s[1][1] : (int)s[1][0];
  return g;
}

template <int BN, int EPI, bool B_MN>
int set_attr(Ctx* c) {
  TB_CUDA(c, cudaFuncSetAttribute(gemm_kernel<BN, EPI, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  GemmCfg<BN, EPI>::SMEM));
  return 0;
}

template <int BN, int EPI, bool B_MN>
int run(Ctx* c, const GemmShape& g, const void* A, const void* B, const void* B2, void* out) {
  CUtensorMap ma, mb, mb2;
  {
    const uint64_t dims[2] = {(uint64_t)g.K, (uint64_t)g.M};
    const uint64_t strides[1] = {(uint64_t)g.K * 2};
    const uint32_t box[2] = {BK, BM};
    if (make_tensor_map(c, &ma, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, A, dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B))
      return 1;
  }
  if (B_MN) {
    const uint64_t dims[2] = {(uint64_t)g.N, (uint64_t)g.K};
    const uint64_t strides[1] = {(uint64_t)g.N * 2};
    const uint32_t box[2] = {64, BK};
    if (make_tensor_map(c, &mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, B, dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B))
      return 1;
    mb2 = mb;
  } else {
    const uint64_t dims[2] = {(uint64_t)g.K, (uint64_t)g.N};
    const uint64_t strides[1] = {(uint64_t)g.K * 2};
    const uint32_t box[2] = {BK, BN};
    if (make_tensor_map(c, &mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, B, dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B))
      return 1;
    mb2 = mb;
    if (EPI == EPI_GATE_UP &&
        make_tensor_map(c, &mb2, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, B2, dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B))
      return 1;
  }
  GemmParams p;
  p.out = out;
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.status = c->status;
  dim3 grid((g.M + BM - 1) / BM, (g.N + BN - 1) / BN);
  gemm_kernel<BN, EPI, B_MN><<<grid, GEMM_THREADS, GemmCfg<BN, EPI>::SMEM, c->stream>>>(ma, mb, mb2, p);
  TB_CUDA(c, cudaGetLastError());
  return 0;
}

template <int EPI, bool B_MN>
int run_plain(Ctx* c, const GemmShape& g, const void* A, const void* B, const void* B2, void* out) {
  dim3 grid((g.N + 31) / 32, (g.M + 31) / 32);
  gemm_plain_kernel<EPI, B_MN><<<grid, 256, 0, c->stream>>>((const __half*)A, (const __half*)B, (const __half*)B2, out,
                                                            g.M, g.N, g.K);
  TB_CUDA(c, cudaGetLastError());
  return 0;
}

int epi_of(Kind k) {
  switch (k) {
    case K_LINEAR:
    case K_MATMUL:
      return EPI_F16;
    case K_LINEAR_RESIDUAL:
      return EPI_RESID;
    case K_GATE_UP:
      return EPI_GATE_UP;
    default:
      return EPI_F32;
  }
}

}  // namespace

// op.p0: 1 = tcgen05 path, 0 = plain path. op.p1: BN.
int make_gemm(Ctx* c, Op& op) {
  const auto& s = op.shapes;
  auto bad = [&](const char* why) { return fail(c, op.name + ": " + why); };
  for (auto& v : s)
    if (v.size() != 2) return bad("every array is two-dimensional");
  const GemmShape g = gemm_shape(op);
  if (op.kind == K_MATMUL) {
    if (s[1][0] != g.K || s[2][0] != g.M || s[2][1] != g.N) return bad("shapes are A[M,K], B[K,N], C[M,N]");
  } else if (op.kind == K_GATE_UP) {
    if (s[1][1] != g.K || s[2] != s[1] || s[3][0] != g.M || s[3][1] != g.N)
      return bad("shapes are X[M,K], Wg[F,K], Wu[F,K], Y[M,F]");
  } else {
    if (s[1][1] != g.K || s[2][0] != g.M || s[2][1] != g.N) return bad("shapes are X[M,K], W[N,K], Y[M,N]");
  }
  if (g.M == 0 || g.N == 0) {
    op.p0 = -1;  // nothing to compute
    return 0;
  }
  const bool tma_ok = g.K > 0 && g.K % 8 == 0 && (op.kind != K_MATMUL || g.N % 8 == 0);
  op.p0 = tma_ok ? 1 : 0;
  if (!tma_ok) return 0;
  // Tile width: wide tiles for prompt-sized M (compute-bound), narrower ones
  // when few rows leave the kernel bound by streaming the weights and the
  // grid has to cover the SMs.
  const int mt = (g.M + BM - 1) / BM;
  int bn;
  if (op.kind == K_GATE_UP) {
    bn = 128;
    if ((long long)mt * ((g.N + 127) / 128) < c->sm_count) bn = 64;
    if ((long long)mt * ((g.N + 63) / 64) < c->sm_count) bn = 32;
  } else if (op.kind == K_MATMUL) {
    bn = 256;
    if ((long long)mt * ((g.N + 255) / 256) < c->sm_count) bn = 128;
    if ((long long)mt * ((g.N + 127) / 128) < c->sm_count) bn = 64;
  } else {
    bn = 256;
    if ((long long)mt * ((g.N + 255) / 256) < c->sm_count) bn = 128;
    if ((long long)mt * ((g.N + 127) / 128) < c->sm_count) bn = 64;
    if ((long long)mt * ((g.N + 63) / 64) < c->sm_count) bn = 32;
  }
  op.p1 = bn;
  int r = 0;
#define TB_ATTR(BN_)                                                        \
  switch (epi_of(op.kind)) {                                                \
    case EPI_F16:                                                           \
      r = op.kind == K_MATMUL ? set_attr<(BN_ < 64 ? 64 : BN_), EPI_F16, true>(c) : set_attr<BN_, EPI_F16, false>(c); \
      break;                                                                \
    case EPI_RESID:                                                         \
      r = set_attr<BN_, EPI_RESID, false>(c);                               \
      break;                                                                \
    case EPI_F32:                                                           \
      r = set_attr<BN_, EPI_F32, false>(c);                                 \
      break;                                                                \
    default:                                                                \
      r = set_attr<(BN_ > 128 ? 128 : BN_), EPI_GATE_UP, false>(c);         \
      break;                                                                \
  }
  switch (bn) {
    case 32: TB_ATTR(32); break;
    case 64: TB_ATTR(64); break;
    case 128: TB_ATTR(128); break;
    default: TB_ATTR(256); break;
  }
#undef TB_ATTR
  return r;
}

int launch_gemm(Ctx* c, Op& op, const uint64_t* a) {
  if (op.p0 < 0) return 0;
  const GemmShape g = gemm_shape(op);
  const void* A = (const void*)a[0];
  const void* B = (const void*)a[1];
  const void* B2 = op.kind == K_GATE_UP ? (const void*)a[2] : nullptr;
  void* out = (void*)a[op.kind == K_GATE_UP ? 3 : 2];
  const int epi = epi_of(op.kind);
  const bool mn = op.kind == K_MATMUL;
  int r = 1;
  if (g.K == 0) {
    // An empty sum: f16/f32 outputs are zero, the residual is unchanged.
    if (epi == EPI_RESID) return 0;
    const size_t bytes = (size_t)g.M * g.N * (epi == EPI_F32 ? 4 : 2);
    TB_CUDA(c, cudaMemsetAsync(out, 0, bytes, c->stream));
    return 0;
  }
  if (op.p0 == 0) {
    if (mn)
      r = run_plain<EPI_F16, true>(c, g, A, B, B2, out);
    else if (epi == EPI_F16)
      r = run_plain<EPI_F16, false>(c, g, A, B, B2, out);
    else if (epi == EPI_RESID)
      r = run_plain<EPI_RESID, false>(c, g, A, B, B2, out);
    else if (epi == EPI_F32)
      r = run_plain<EPI_F32, false>(c, g, A, B, B2, out);
    else
      r = run_plain<EPI_GATE_UP, false>(c, g, A, B, B2, out);
  } else {
#define TB_RUN(BN_)                                                                                  \
  if (mn)                                                                                            \
    r = run<(BN_ < 64 ? 64 : BN_), EPI_F16, true>(c, g, A, B, B2, out);                              \
  else if (epi == EPI_F16)                                                                           \
    r = run<BN_, EPI_F16, false>(c, g, A, B, B2, out);                                               \
  else if (epi == EPI_RESID)                                                                         \
    r = run<BN_, EPI_RESID, false>(c, g, A, B, B2, out);                                             \
  else if (epi == EPI_F32)                                                                           \
    r = run<BN_, EPI_F32, false>(c, g, A, B, B2, out);                                               \
  else                                                                                               \
    r = run<(BN_ > 128 ? 128 : BN_), EPI_GATE_UP, false>(c, g, A, B, B2, out);
    switch (op.p1) {
      case 32: TB_RUN(32); break;
      case 64: TB_RUN(64); break;
      case 128: TB_RUN(128); break;
      default: TB_RUN(256); break;
    }
#undef TB_RUN
  }
  if (r) return r;
  c->launches += 1;
  return 0;
}

}  // namespace tb
