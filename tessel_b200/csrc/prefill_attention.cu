// Causal FlashAttention over the tokens of a step:
//   prefill_attention  packed GQA, Q/O [S,H,D], K/V [S,G,D], per-row `starts`
//                      (kernels/llm.tl:116-145)
//   flash_attention    Q/K/V/O [H,S,D]            (kernels/attention.tl:4-24)
//
// tcgen05 path (D in {64, 128}): one CTA owns 128 query rows of one head. A
// producer warp brings the Q tile once and then 128-key K and V tiles through
// a two-stage TMA ring. One thread issues the MMAs: S = Q K^T (M 128, N 128)
// into tensor memory, and O_blk = P V (M 128, N D) once the softmax warps have
// published P. Four softmax warps own one query row per thread: they read S
// out of tensor memory, apply scale and the causal / sequence-start mask, keep
// the online maximum and sum, round P to f16 into swizzled shared memory (the
// A operand of the second MMA, as kernels/llm.tl:143 rounds it), then fold
// O_blk into their f32 accumulator row. The S MMA of the next key block is
// issued right behind the P V MMA, so it runs while the softmax warps fold.
//
// The key loop starts at starts[first row of the block] (not tile aligned) and
// the running maximum starts at -1e30, as the reference's does.
//
// Generic path (any D that is a multiple of 8): one warp per (row, head).
#include "common.cuh"

namespace tb {

namespace {

constexpr int FA_BM = 128, FA_BN = 128;
constexpr int FA_THREADS = 192;
constexpr float LOG2E = 1.4426950408889634f;

struct FaParams {
  const int* starts;  // null for the plain layout
  __half* O;
  float scale;
  int S, H, G, plain;
  unsigned int* status;
};

template <int D>
struct FaSmem {
  static constexpr int SUB = D / 64;
  static constexpr int Q_BYTES = FA_BM * D * 2;
  static constexpr int KV_BYTES = FA_BN * D * 2;      // one K (or V) tile
  static constexpr int STAGE = 2 * KV_BYTES;
  static constexpr int P_BYTES = FA_BM * FA_BN * 2;
  static constexpr int OFF_KV = Q_BYTES;
  static constexpr int OFF_P = OFF_KV + 2 * STAGE;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int TOTAL = OFF_BAR + 16 * 8 + 1024;
  static constexpr int TMEM_COLS = 256;  // S: [0,128), O_blk: [128, 128 + D)
};

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
    fa_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
              const __grid_constant__ CUtensorMap mapV, const FaParams p) {
  using SM = FaSmem<D>;
  constexpr int SUB = SM::SUB;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + SM::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_full = bars + 7;
  uint64_t* o_free = bars + 8;
  uint32_t* tmem_slot = (uint32_t*)(bars + 9);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i0 = blockIdx.x * FA_BM, h = blockIdx.y;
  const int g = p.plain ? h : h / (p.H / p.G);
  const int lo = p.starts ? p.starts[i0] : 0;
  const int hi = min(i0 + FA_BM, p.S);
  const int nblk = (hi - lo + FA_BN - 1) / FA_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(&kv_full[0], 1);
    mbar_init(&kv_full[1], 1);
    mbar_init(&kv_empty[0], 1);
    mbar_init(&kv_empty[1], 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    mbar_init(o_free, 128);
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, SM::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_s = tmem, tmem_o = tmem + 128;

  if (warp == 4) {
    if (elect_one()) {
      prefetch_tmap(&mapQ);
      prefetch_tmap(&mapK);
      prefetch_tmap(&mapV);
      mbar_expect_tx(q_full, SM::Q_BYTES);
#pragma unroll
      for (int sub = 0; sub < SUB; ++sub) {
        if (p.plain)
          tma_load_3d(smem + sub * (FA_BM * 128), &mapQ, q_full, sub * 64, i0, h);
        else
          tma_load_3d(smem + sub * (FA_BM * 128), &mapQ, q_full, sub * 64, h, i0);
      }
      for (int jb = 0; jb < nblk; ++jb) {
        const int s = jb & 1, k = jb >> 1;
        const int key0 = lo + jb * FA_BN;
        mbar_wait(&kv_empty[s], (k & 1) ^ 1, p.status, 301);
        mbar_expect_tx(&kv_full[s], SM::STAGE);
        unsigned char* kd = smem + SM::OFF_KV + s * SM::STAGE;
        unsigned char* vd = kd + SM::KV_BYTES;
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
          if (p.plain) {
            tma_load_3d(kd + sub * (FA_BN * 128), &mapK, &kv_full[s], sub * 64, key0, g);
            tma_load_3d(vd + sub * (FA_BN * 128), &mapV, &kv_full[s], sub * 64, key0, g);
          } else {
            tma_load_3d(kd + sub * (FA_BN * 128), &mapK, &kv_full[s], sub * 64, g, key0);
            tma_load_3d(vd + sub * (FA_BN * 128), &mapV, &kv_full[s], sub * 64, g, key0);
          }
        }
      }
    }
  } else if (warp == 5) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_f16(FA_BM, FA_BN, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_f16(FA_BM, D, 0, 1);
      const uint32_t qa = smem_u32(smem);
      const uint32_t pa = smem_u32(smem + SM::OFF_P);
      mbar_wait(q_full, 0, p.status, 302);
      for (int jb = 0; jb < nblk; ++jb) {
        const int s = jb & 1, k = jb >> 1;
        const uint32_t ka = smem_u32(smem + SM::OFF_KV + s * SM::STAGE);
        const uint32_t va = ka + SM::KV_BYTES;
        mbar_wait(&kv_full[s], k & 1, p.status, 303);
        tc_fence_after();
#pragma unroll
        for (int kd = 0; kd < D / 16; ++kd) {
          const uint32_t off = (kd >> 2) * (FA_BM * 128) + (kd & 3) * 32;
          umma_f16(tmem_s, umma_desc_sw128(qa + off, 16, 1024), umma_desc_sw128(ka + off, 16, 1024), idesc_s,
                   kd > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        mbar_wait(p_full, jb & 1, p.status, 304);
        if (jb > 0) mbar_wait(o_free, (jb - 1) & 1, p.status, 305);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < FA_BN / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * (FA_BM * 128) + (kk & 3) * 32;
          umma_f16(tmem_o, umma_desc_sw128(pa + aoff, 16, 1024),
                   umma_desc_sw128(va + kk * 2048, FA_BN * 128, 1024), idesc_o, kk > 0 ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(&kv_empty[s]);
      }
    }
  } else {
    // ---- softmax warps: thread = query row, TMEM lanes 32*warp .. +31 -------
    const int r = threadIdx.x;  // 0..127
    const int row = i0 + r;
    const int st = (p.starts && row < p.S) ? p.starts[row] : 0;
    const float sc2 = p.scale * LOG2E;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    unsigned char* prow = smem + SM::OFF_P + r * 128;
    float m = -1e30f, l = 0.f;
    float acc[D];
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    for (int jb = 0; jb < nblk; ++jb) {
      const int key0 = lo + jb * FA_BN;
      mbar_wait(s_full, jb & 1, p.status, 306);
      tc_fence_after();
      // Pass 1: the block's row maximum (log2 domain).
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_s + lane_base + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = key0 + c0 + j;
          const bool ok = col <= row && col >= st && col < p.S;
          mx = fmaxf(mx, ok ? __uint_as_float(v[j]) * sc2 : -INFINITY);
        }
      }
      const float m2 = fmaxf(m, mx);
      // Pass 2: probabilities, rounded to f16 into the swizzled P tile.
      float sum = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_s + lane_base + c0, v);
        tmem_ld_wait();
        float pr[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = key0 + c0 + j;
          const bool ok = col <= row && col >= st && col < p.S;
          pr[j] = ok ? exp2f(__uint_as_float(v[j]) * sc2 - m2) : 0.f;
          sum += pr[j];
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int c = (c0 >> 3) + ch;  // 16-byte chunk along the keys, 0..15
          uint4 o;
          o.x = pack_h2(pr[ch * 8 + 0], pr[ch * 8 + 1]);
          o.y = pack_h2(pr[ch * 8 + 2], pr[ch * 8 + 3]);
          o.z = pack_h2(pr[ch * 8 + 4], pr[ch * 8 + 5]);
          o.w = pack_h2(pr[ch * 8 + 6], pr[ch * 8 + 7]);
          *reinterpret_cast<uint4*>(prow + (c >> 3) * (FA_BM * 128) + (((c & 7) ^ (r & 7)) << 4)) = o;
        }
      }
      const float a = exp2f(m - m2);
      l = l * a + sum;
      m = m2;
      tc_fence_before();
      fence_proxy_async();  // P must be visible to the tensor core's reads
      mbar_arrive(p_full);
      mbar_wait(o_full, jb & 1, p.status, 307);
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_o + lane_base + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c0 + j] = acc[c0 + j] * a + __uint_as_float(v[j]);
      }
      tc_fence_before();
      mbar_arrive(o_free);
    }
    if (row < p.S) {
      const float inv = 1.0f / l;
      __half* o = p.plain ? p.O + ((size_t)h * p.S + row) * D : p.O + ((size_t)row * p.H + h) * D;
#pragma unroll
      for (int d = 0; d < D; d += 8) {
        uint4 w;
        w.x = pack_h2(acc[d] * inv, acc[d + 1] * inv);
        w.y = pack_h2(acc[d + 2] * inv, acc[d + 3] * inv);
        w.z = pack_h2(acc[d + 4] * inv, acc[d + 5] * inv);
        w.w = pack_h2(acc[d + 6] * inv, acc[d + 7] * inv);
        *reinterpret_cast<uint4*>(o + d) = w;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, SM::TMEM_COLS);
  }
}

// Generic path: one warp per (row, head), keys visited one at a time.
__global__ void fa_generic_kernel(const __half* __restrict__ Q, const __half* __restrict__ K,
                                  const __half* __restrict__ V, const int* __restrict__ starts, __half* __restrict__ O,
                                  float scale, int S, int H, int G, int D, int plain) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)S * H) return;
  const int row = (int)(w / H), h = (int)(w % H);
  const int g = plain ? h : h / (H / G);
  const size_t qs = plain ? (size_t)D : (size_t)H * D, qh = plain ? (size_t)S * D : (size_t)D;
  const size_t ks = plain ? (size_t)D : (size_t)G * D, kh = plain ? (size_t)S * D : (size_t)D;
  constexpr int MAXC = 8;
  float q[MAXC], acc[MAXC];
  for (int c = 0; c < MAXC; ++c) {
    const int d = lane + 32 * c;
    q[c] = d < D ? __half2float(Q[row * qs + h * qh + d]) : 0.f;
    acc[c] = 0.f;
  }
  const int st = starts ? starts[row] : 0;
  float m = -1e30f, l = 0.f;
  for (int col = st; col <= row; ++col) {
    const __half* kr = K + col * ks + g * kh;
    const __half* vr = V + col * ks + g * kh;
    float s = 0.f;
    for (int c = 0; c < MAXC; ++c) {
      const int d = lane + 32 * c;
      if (d < D) s += q[c] * __half2float(kr[d]);
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    s *= scale;
    const float m2 = fmaxf(m, s);
    const float a = expf(m - m2);
    const float pr = expf(s - m2);
    const float p16 = __half2float(__float2half_rn(pr));
    l = l * a + pr;
    for (int c = 0; c < MAXC; ++c) {
      const int d = lane + 32 * c;
      if (d < D) acc[c] = acc[c] * a + p16 * __half2float(vr[d]);
    }
    m = m2;
  }
  for (int c = 0; c < MAXC; ++c) {
    const int d = lane + 32 * c;
    if (d < D) O[row * qs + h * qh + d] = __float2half_rn(acc[c] / l);
  }
}

struct FaShape {
  int S, H, G, D, plain;
};

FaShape fa_shape(const Op& op) {
  const auto& s = op.shapes;
  FaShape f;
  f.plain = op.kind == K_FLASH_ATTENTION;
  if (f.plain) {
    f.H = (int)s[0][0];
    f.S = (int)s[0][1];
    f.D = (int)s[0][2];
    f.G = f.H;
  } else {
    f.S = (int)s[0][0];
    f.H = (int)s[0][1];
    f.D = (int)s[0][2];
    f.G = (int)s[1][1];
  }
  return f;
}

template <int D>
int run_fa(Ctx* c, const FaShape& f, const void* Q, const void* K, const void* V, const int* starts, void* O,
           float scale) {
  CUtensorMap mq, mk, mv;
  auto mk_map = [&](CUtensorMap* m, const void* base, int heads) {
    if (f.plain) {
      const uint64_t dims[3] = {(uint64_t)D, (uint64_t)f.S, (uint64_t)heads};
      const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)f.S * D * 2};
      const uint32_t box[3] = {64, 128, 1};
      return make_tensor_map(c, m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    }
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)heads, (uint64_t)f.S};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)heads * D * 2};
    const uint32_t box[3] = {64, 1, 128};
    return make_tensor_map(c, m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
  };
  if (mk_map(&mq, Q, f.H) || mk_map(&mk, K, f.G) || mk_map(&mv, V, f.G)) return 1;
  FaParams p;
  p.starts = starts;
  p.O = (__half*)O;
  p.scale = scale;
  p.S = f.S;
  p.H = f.H;
  p.G = f.G;
  p.plain = f.plain;
  p.status = c->status;
  dim3 grid((f.S + FA_BM - 1) / FA_BM, f.H);
  fa_kernel<D><<<grid, FA_THREADS, FaSmem<D>::TOTAL, c->stream>>>(mq, mk, mv, p);
  TB_CUDA(c, cudaGetLastError());
  return 0;
}

}  // namespace

int make_prefill(Ctx* c, Op& op) {
  const auto& s = op.shapes;
  auto bad = [&](const char* why) { return fail(c, op.name + ": " + why); };
  if (op.kind == K_FLASH_ATTENTION) {
    if (s[0].size() != 3 || s[1] != s[0] || s[2] != s[0] || s[3] != s[0]) return bad("shapes are Q,K,V,O [H,S,D]");
  } else {
    if (s[0].size() != 3 || s[1].size() != 3 || s[2] != s[1] || s[4] != s[0] || s[3].size() != 1 ||
        s[3][0] != s[0][0] || s[1][0] != s[0][0] || s[1][2] != s[0][2])
      return bad("shapes are Q[S,H,D], K[S,G,D], V[S,G,D], starts[S], O[S,H,D]");
  }
  const FaShape f = fa_shape(op);
  if (f.G < 1 || f.H % f.G) return bad("heads must be a multiple of kv heads");
  if (f.D % 8 || f.D > 256) return bad("head_dim must be a multiple of 8, at most 256");
  op.p0 = (f.D == 64 || f.D == 128) && f.S > 0 ? 1 : 0;
  if (op.p0) {
    if (f.D == 128)
      TB_CUDA(c, cudaFuncSetAttribute(fa_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaSmem<128>::TOTAL));
    else
      TB_CUDA(c, cudaFuncSetAttribute(fa_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaSmem<64>::TOTAL));
  }
  return 0;
}

int launch_prefill(Ctx* c, Op& op, const uint64_t* a) {
  const FaShape f = fa_shape(op);
  if (f.S == 0 || f.H == 0) return 0;
  const void *Q = (const void*)a[0], *K = (const void*)a[1], *V = (const void*)a[2];
  const int* starts = f.plain ? nullptr : (const int*)a[3];
  void* O = (void*)a[f.plain ? 3 : 4];
  const float scale = bits_f32(a[f.plain ? 4 : 5]);
  int r;
  if (op.p0) {
    r = f.D == 128 ? run_fa<128>(c, f, Q, K, V, starts, O, scale) : run_fa<64>(c, f, Q, K, V, starts, O, scale);
  } else {
    const long long warps = (long long)f.S * f.H;
    fa_generic_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, c->stream>>>((const __half*)Q, (const __half*)K,
                                                                          (const __half*)V, starts, (__half*)O, scale,
                                                                          f.S, f.H, f.G, f.D, f.plain);
    cudaError_t e = cudaGetLastError();
    r = e == cudaSuccess ? 0 : cuda_fail(c, e, "fa_generic_kernel");
  }
  if (r) return r;
  c->launches += 1;
  return 0;
}

}  // namespace tb
