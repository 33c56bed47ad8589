// Paged grouped-query decode attention (kernels/llm.tl:150-172; with G == H it
// is kernels/attention.tl:29-51).
//
// One query token per sequence attends to its paged KV cache
// [pages, P, G, D]. The reference launches one warp per (sequence, query
// head), so each of the H/G query heads of a KV head re-reads the same pages.
// Here one CTA serves ALL query heads of a KV head, so every page crosses HBM
// once. When that gives too few CTAs to fill the SMs, the key range is split
// over CTAs (split-KV) and the partials are merged by a second, tiny kernel;
// otherwise the one kernel writes the output itself.
//
// Fast path (P == 16, D in {64, 128}, f16): a producer warp walks the block
// table and streams (page, kv-head) tiles into a shared-memory ring with TMA
// (128-byte swizzle, mbarrier completion); four consumer warps take pages
// round-robin, compute K q^T and P^T-weighted V sums on mma.sync m16n8k16
// tiles (tokens ride M, the <= 8 query heads of the group ride N), and keep an
// online softmax whose row reductions are warp shuffles. Probabilities are fed
// to the second product as a two-term f16 split (hi + lo), which keeps the
// product at f32-level accuracy although the reference never rounds p to f16.
//
// Generic path: any P and D (multiple of 8), one warp per (sequence, head),
// CUDA-core dot products; it is the reference's own schedule.
#include "common.cuh"

namespace tb {

namespace {

constexpr int DEC_WARPS = 4;                    // consumer warps
constexpr int DEC_THREADS = (DEC_WARPS + 1) * 32;  // + one producer warp
#ifndef TB_DEC_STAGES
#define TB_DEC_STAGES 8
#endif
constexpr int DEC_STAGES = TB_DEC_STAGES;                   // pages in flight per CTA
constexpr float LOG2E = 1.4426950408889634f;
// Consumer warp w takes pages w, w + DEC_WARPS, ...: with a ring depth that is a multiple of
// DEC_WARPS a slot is always read by the same warp, which therefore waits for every one of the
// slot's phases in turn. Any other depth would let a warp skip a phase of a slot, and a parity
// test cannot tell a phase from the one two before it.
static_assert(DEC_STAGES % DEC_WARPS == 0, "ring depth must be a multiple of the consumer warps");

struct DecodeParams {
  const __half* Q;
  const int* table;
  const int* lens;
  __half* O;
  float* part_acc;  // [B, H, nsplit, D]
  float* part_ml;   // [B, H, nsplit, 2]
  float scale;
  int B, H, G, NP, MP, chunk, nsplit;
  unsigned int* status;
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movm_t(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared memory of the fast path, 1024-byte aligned: DEC_STAGES stages of
// [K tile][V tile], each tile D/64 sub-tiles of 16 rows x 128 bytes.
template <int D>
struct DecSmem {
  static constexpr int SUB = D / 64;
  static constexpr int TILE = SUB * 16 * 128;  // bytes of one K (or V) page tile
  static constexpr int STAGE = 2 * TILE;
  static constexpr int RING = DEC_STAGES * STAGE;
  static constexpr int MERGE = DEC_WARPS * (8 * D + 16) * 4;  // per-warp acc[8][D], m[8], l[8]
  static constexpr int BARS = RING > MERGE ? RING : MERGE;    // offset of the barriers
  static constexpr int TOTAL = BARS + 2 * DEC_STAGES * 8 + 1024;  // + alignment slack
};

template <int D>
__global__ void __launch_bounds__(DEC_THREADS) decode_tma_kernel(const __grid_constant__ CUtensorMap mapK,
                                                                 const __grid_constant__ CUtensorMap mapV,
                                                                 const DecodeParams p) {
  pdl_launch();
  pdl_wait();
  using SM = DecSmem<D>;
  constexpr int SUB = SM::SUB;
  constexpr int P = 16;
  const int split = blockIdx.x;
  const int hgroups = (p.H / p.G + 7) / 8;
  const int g = blockIdx.y / hgroups, hg = blockIdx.y % hgroups;
  const int b = blockIdx.z;
  const int n = p.lens[b];
  const int npages = (n + P - 1) / P;
  const int first = split * p.chunk;
  if (n <= 0) {
    // No cached token: the reference's 0/0 (kernels/llm.tl:172 with l == 0).
    if (p.nsplit == 1) {
      const int hq0 = p.H / p.G, hb = g * hq0 + hg * 8, nhb = min(8, hq0 - hg * 8);
      for (int i = threadIdx.x; i < nhb * D; i += blockDim.x)
        p.O[((size_t)b * p.H + hb + i / D) * D + i % D] = __float2half_rn(__int_as_float(0x7fc00000));
    }
    return;
  }
  if (first >= npages) return;  // uniform for the CTA: nothing to do
  // A length that runs past the block table (lens > MP * 16) is not an error in the reference:
  // its masked table load reads 0 there, so those tokens see page 0. The last split takes them.
  const int count = split == p.nsplit - 1 ? npages - first : min(p.chunk, npages - first);

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + SM::BARS);
  uint64_t* empty = full + DEC_STAGES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < DEC_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    fence_barrier_init();
  }
  __syncthreads();

  const int hq = p.H / p.G;                   // query heads per kv head
  const int h0 = g * hq + hg * 8;             // first query head of this CTA
  const int nh = min(8, hq - hg * 8);         // query heads served here

  if (warp == DEC_WARPS) {
    // ---- producer: block-table walk + TMA issue ---------------------------
    if (lane == 0) {
      prefetch_tmap(&mapK);
      prefetch_tmap(&mapV);
    }
    for (int j0 = 0; j0 < count; j0 += 32) {
      const int col = first + j0 + lane;  // beyond the table: page 0, as a masked load gives
      const int mine = (j0 + lane < count && col < p.MP) ? p.table[(size_t)b * p.MP + col] : 0;
      const int lim = min(32, count - j0);
      for (int i = 0; i < lim; ++i) {
        const int page = __shfl_sync(0xffffffffu, mine, i);
        if (lane == 0) {
          const int j = j0 + i, s = j % DEC_STAGES, k = j / DEC_STAGES;
          mbar_wait(&empty[s], (k & 1) ^ 1, p.status, 101);
          mbar_expect_tx(&full[s], SM::STAGE);
          unsigned char* dst = smem + s * SM::STAGE;
#pragma unroll
          for (int sub = 0; sub < SUB; ++sub) {
            tma_load_4d(dst + sub * 2048, &mapK, &full[s], 0, g * SUB + sub, 0, page);
            tma_load_4d(dst + SM::TILE + sub * 2048, &mapV, &full[s], 0, g * SUB + sub, 0, page);
          }
        }
      }
    }
    return;
  }

  // ---- consumers -----------------------------------------------------------
  const int gq = lane >> 2, t = lane & 3;
  // Q^T fragments (B operand of K q^T): b0 = Q[head gq][16kd + 2t, +1], b1 = same + 8.
  uint32_t qf[D / 16][2];
  {
    const bool live = gq < nh;
    const __half* q = p.Q + ((size_t)b * p.H + h0 + (live ? gq : 0)) * D;
#pragma unroll
    for (int kd = 0; kd < D / 16; ++kd) {
      qf[kd][0] = live ? *reinterpret_cast<const uint32_t*>(q + kd * 16 + 2 * t) : 0u;
      qf[kd][1] = live ? *reinterpret_cast<const uint32_t*>(q + kd * 16 + 8 + 2 * t) : 0u;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float acc[D / 16][4];
#pragma unroll
  for (int i = 0; i < D / 16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  const int mi = lane >> 3, rin = lane & 7;
  // ldmatrix row of this lane for the K tile (A of K q^T) and the V tile (A of V^T P^T).
  const int k_tok = rin + (mi & 1) * 8, k_dsel = mi >> 1;
  const int v_tok = rin + (mi >> 1) * 8, v_dsel = mi & 1;
  const float sc2 = p.scale * LOG2E;  // scores are kept in the log2 domain

  for (int j = warp; j < count; j += DEC_WARPS) {
    const int s = j % DEC_STAGES, k = j / DEC_STAGES;
    mbar_wait(&full[s], k & 1, p.status, 102);
    const uint32_t kb = smem_u32(smem + s * SM::STAGE);
    const uint32_t vb = kb + SM::TILE;

    float sfr[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kd = 0; kd < D / 16; ++kd) {
      const int ch = 2 * kd + k_dsel;  // 16-byte chunk along D
      const uint32_t addr = kb + (ch >> 3) * 2048 + k_tok * 128 + (((ch & 7) ^ (k_tok & 7)) << 4);
      uint32_t a0, a1, a2, a3;
      ldsm_x4(addr, a0, a1, a2, a3);
      mma16816(sfr, a0, a1, a2, a3, qf[kd][0], qf[kd][1]);
    }
    // sfr[0..1]: token gq, heads 2t, 2t+1; sfr[2..3]: token gq + 8.
    const int tok0 = (first + j) * P + gq;
    const bool ok0 = tok0 < n, ok1 = tok0 + 8 < n;
    float s00 = ok0 ? sfr[0] * sc2 : -INFINITY, s01 = ok0 ? sfr[1] * sc2 : -INFINITY;
    float s10 = ok1 ? sfr[2] * sc2 : -INFINITY, s11 = ok1 ? sfr[3] * sc2 : -INFINITY;
    float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    // Token 0 of a page is always inside the sequence, so mx is finite.
    const float m20 = fmaxf(m[0], mx0), m21 = fmaxf(m[1], mx1);
    const float a0s = exp2f(m[0] - m20), a1s = exp2f(m[1] - m21);
    const float p00 = exp2f(s00 - m20), p01 = exp2f(s01 - m21);
    const float p10 = exp2f(s10 - m20), p11 = exp2f(s11 - m21);
    l[0] = l[0] * a0s + (p00 + p10);
    l[1] = l[1] * a1s + (p01 + p11);
    m[0] = m20;
    m[1] = m21;
    // p = hi + lo in f16; P^T fragments through an 8x8 transpose.
    const __half2 h0p = __floats2half2_rn(p00, p01), h1p = __floats2half2_rn(p10, p11);
    const float2 f0 = __half22float2(h0p), f1 = __half22float2(h1p);
    const uint32_t lo0 = pack_h2(p00 - f0.x, p01 - f0.y), lo1 = pack_h2(p10 - f1.x, p11 - f1.y);
    const uint32_t bh0 = movm_t(*reinterpret_cast<const uint32_t*>(&h0p));
    const uint32_t bh1 = movm_t(*reinterpret_cast<const uint32_t*>(&h1p));
    const uint32_t bl0 = movm_t(lo0), bl1 = movm_t(lo1);
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) {
      acc[mt][0] *= a0s;
      acc[mt][1] *= a1s;
      acc[mt][2] *= a0s;
      acc[mt][3] *= a1s;
      const int ch = 2 * mt + v_dsel;
      const uint32_t addr = vb + (ch >> 3) * 2048 + v_tok * 128 + (((ch & 7) ^ (v_tok & 7)) << 4);
      uint32_t a0, a1, a2, a3;
      ldsm_x4_t(addr, a0, a1, a2, a3);
      mma16816(acc[mt], a0, a1, a2, a3, bh0, bh1);
      mma16816(acc[mt], a0, a1, a2, a3, bl0, bl1);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }

  // Sum l over the token lanes; m is already uniform over them.
#pragma unroll
  for (int o = 4; o <= 16; o <<= 1) {
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], o);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], o);
  }

  // ---- merge the four warps (the ring is idle: every issued page was consumed)
  asm volatile("bar.sync 1, %0;" ::"r"(DEC_WARPS * 32) : "memory");
  float* wacc = (float*)smem + warp * (8 * D + 16);  // acc[head][d], then m[8], l[8]
#pragma unroll
  for (int mt = 0; mt < D / 16; ++mt) {
    wacc[(2 * t) * D + mt * 16 + gq] = acc[mt][0];
    wacc[(2 * t + 1) * D + mt * 16 + gq] = acc[mt][1];
    wacc[(2 * t) * D + mt * 16 + gq + 8] = acc[mt][2];
    wacc[(2 * t + 1) * D + mt * 16 + gq + 8] = acc[mt][3];
  }
  if (gq == 0) {
    wacc[8 * D + 2 * t] = m[0];
    wacc[8 * D + 2 * t + 1] = m[1];
    wacc[8 * D + 8 + 2 * t] = l[0];
    wacc[8 * D + 8 + 2 * t + 1] = l[1];
  }
  asm volatile("bar.sync 1, %0;" ::"r"(DEC_WARPS * 32) : "memory");
  const float* base = (const float*)smem;
  for (int i = threadIdx.x; i < nh * D; i += DEC_WARPS * 32) {
    const int hh = i / D, d = i % D;
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mt = fmaxf(mt, base[w * (8 * D + 16) + 8 * D + hh]);
    float lt = 0.f, at = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = base[w * (8 * D + 16) + 8 * D + hh];
      const float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - mt);
      lt += base[w * (8 * D + 16) + 8 * D + 8 + hh] * wgt;
      at += base[w * (8 * D + 16) + hh * D + d] * wgt;
    }
    if (p.nsplit == 1) {
      // The launch has one split per sequence: no partial to merge, no second kernel.
      p.O[((size_t)b * p.H + h0 + hh) * D + d] = __float2half_rn(at / lt);
      continue;
    }
    const size_t o = ((size_t)b * p.H + h0 + hh) * p.nsplit + split;
    p.part_acc[o * D + d] = at;
    if (d == 0) {
      p.part_ml[o * 2] = mt;
      p.part_ml[o * 2 + 1] = lt;
    }
  }
}

// Merges the split partials of one (sequence, head): O = f16(sum_s acc_s w_s / sum_s l_s w_s).
// A sequence with lens == 0 has no partial and gives 0/0 = NaN, as the
// reference does (kernels/llm.tl:172 with l == 0).
// One warp per (sequence, head), eight per block; a lane owns D/32 consecutive columns.
__global__ void decode_combine_kernel(const DecodeParams p, int D, int P) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (bh >= p.B * p.H) return;
  const int b = bh / p.H;
  const int n = p.lens[b];
  const int npages = n > 0 ? (n + P - 1) / P : 0;
  const int ns = min((npages + p.chunk - 1) / p.chunk, p.nsplit);  // the last split takes what runs past the table
  const float* ml = p.part_ml + (size_t)bh * p.nsplit * 2;
  float mt = -INFINITY;
  for (int s = lane; s < ns; s += 32) mt = fmaxf(mt, ml[s * 2]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
  const int V = D >> 5;  // 2 or 4 on the paths that use this kernel
  const float* acc = p.part_acc + (size_t)bh * p.nsplit * D + lane * V;
  float lt = 0.f, at[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < ns; ++s) {
    const float w = exp2f(ml[s * 2] - mt);
    lt += ml[s * 2 + 1] * w;
    if (V == 4) {
      const float4 a = *reinterpret_cast<const float4*>(acc + (size_t)s * D);
      at[0] += a.x * w, at[1] += a.y * w, at[2] += a.z * w, at[3] += a.w * w;
    } else {
      const float2 a = *reinterpret_cast<const float2*>(acc + (size_t)s * D);
      at[0] += a.x * w, at[1] += a.y * w;
    }
  }
  __half* o = p.O + (size_t)bh * D + lane * V;
  if (V == 4) {
    uint2 y;
    y.x = pack_h2(at[0] / lt, at[1] / lt);
    y.y = pack_h2(at[2] / lt, at[3] / lt);
    *reinterpret_cast<uint2*>(o) = y;
  } else {
    *reinterpret_cast<uint32_t*>(o) = pack_h2(at[0] / lt, at[1] / lt);
  }
}

// Generic path: one warp per (sequence, head); lane owns D/32-strided columns.
__global__ void decode_generic_kernel(const __half* __restrict__ Q, const __half* __restrict__ Kc,
                                      const __half* __restrict__ Vc, const int* __restrict__ table,
                                      const int* __restrict__ lens, __half* __restrict__ O, float scale, int B, int H,
                                      int G, int D, int NP, int P, int MP) {
  pdl_launch();
  pdl_wait();
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= B * H) return;
  const int b = w / H, h = w % H, g = h / (H / G);
  const int n = lens[b];
  constexpr int MAXC = 8;  // columns per lane: D <= 256
  float q[MAXC], acc[MAXC];
  for (int i = 0; i < MAXC; ++i) {
    const int d = lane + 32 * i;
    q[i] = d < D ? __half2float(Q[((size_t)b * H + h) * D + d]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int t0 = 0; t0 < n; t0 += P) {
    const int col = t0 / P;
    const int page = col < MP ? table[(size_t)b * MP + col] : 0;
    const bool in = page >= 0 && page < NP;
    for (int i = 0; i < P && t0 + i < n; ++i) {
      const __half* kr = Kc + (((size_t)(in ? page : 0) * P + i) * G + g) * D;
      const __half* vr = Vc + (((size_t)(in ? page : 0) * P + i) * G + g) * D;
      float s = 0.f;
      for (int c = 0; c < MAXC; ++c) {
        const int d = lane + 32 * c;
        if (d < D && in) s += __half2float(kr[d]) * q[c];
      }
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      s *= scale;
      const float m2 = fmaxf(m, s);
      const float a = expf(m - m2), pr = expf(s - m2);
      l = l * a + pr;
      for (int c = 0; c < MAXC; ++c) {
        const int d = lane + 32 * c;
        const float v = (d < D && in) ? __half2float(vr[d]) : 0.f;
        acc[c] = acc[c] * a + pr * v;
      }
      m = m2;
    }
  }
  for (int c = 0; c < MAXC; ++c) {
    const int d = lane + 32 * c;
    if (d < D) O[((size_t)b * H + h) * D + d] = __float2half_rn(acc[c] / l);
  }
}

struct DecodeShape {
  int B, H, G, D, NP, P, MP;
};

DecodeShape shape_of(const Op& op) {
  const auto& s = op.shapes;
  DecodeShape d;
  d.B = (int)s[0][0];
  d.H = (int)s[0][1];
  d.D = (int)s[0][2];
  d.NP = (int)s[1][0];
  d.P = (int)s[1][1];
  d.G = (int)s[1][2];
  d.MP = (int)s[3][1];
  return d;
}

}  // namespace

int make_decode(Ctx* c, Op& op) {
  const auto& s = op.shapes;
  auto bad = [&](const char* why) { return fail(c, op.name + ": " + why); };
  if (s[0].size() != 3 || s[1].size() != 4 || s[2] != s[1] || s[3].size() != 2 || s[4].size() != 1 || s[5] != s[0])
    return bad("shapes are Q[B,H,D], Kc[NP,P,G,D], Vc[NP,P,G,D], table[B,MP], lens[B], O[B,H,D]");
  DecodeShape d = shape_of(op);
  if (s[1][3] != d.D || s[3][0] != d.B || s[4][0] != d.B) return bad("shapes disagree");
  if (d.G < 1 || d.H % d.G) return bad("heads must be a multiple of kv heads");
  if (d.D % 8 || d.D > 256) return bad("head_dim must be a multiple of 8, at most 256");
  const bool fast = d.P == 16 && (d.D == 64 || d.D == 128) && d.B > 0 && d.NP > 0 && d.MP > 0;
  op.p0 = fast ? 1 : 0;
  if (!fast) return 0;
  // Split-KV: aim at ~4 CTAs per SM, chunks a multiple of the consumer warps.
  const int hgroups = (d.H / d.G + 7) / 8;
  const long long units = (long long)d.B * d.G * hgroups;
  long long want = (4LL * c->sm_count + units - 1) / units;
  if (const char* e = getenv("TB200_DECODE_SPLITS")) {  // tuning and tests; a value that is not a count is an error
    char* end = nullptr;
    const long v = strtol(e, &end, 10);
    if (end == e || *end != 0 || v < 1 || v > 4096) return bad("TB200_DECODE_SPLITS must be a positive integer");
    want = v;
  }
  int max_split = (d.MP + 3) / 4;
  // Once every SM has a CTA or two anyway, more splits only shorten the tail, and a split costs
  // its start-up (barriers, the first pages' latency) and a partial to merge: measured at 256
  // sequences x 1 KV head (an 8-way tensor-parallel rank), two splits of 72 pages take 51 us,
  // three of 48 pages 57 us, one 58 us. So there chunks stay 64 pages or longer.
  if (units * 2 >= 3LL * c->sm_count && !getenv("TB200_DECODE_SPLITS")) max_split = d.MP >= 128 ? d.MP / 64 : 1;
  int nsplit = (int)(want < 1 ? 1 : (want > max_split ? max_split : want));
  int chunk = (d.MP + nsplit - 1) / nsplit;
  chunk = (chunk + 3) / 4 * 4;
  nsplit = (d.MP + chunk - 1) / chunk;
  op.p1 = chunk;
  op.p2 = nsplit;
  op.scratch_bytes = (size_t)d.B * d.H * nsplit * (d.D + 2) * sizeof(float);
  TB_CUDA(c, cudaMalloc(&op.scratch, op.scratch_bytes));
  const int smem = d.D == 128 ? DecSmem<128>::TOTAL : DecSmem<64>::TOTAL;
  if (d.D == 128)
    TB_CUDA(c, cudaFuncSetAttribute(decode_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  else
    TB_CUDA(c, cudaFuncSetAttribute(decode_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  return 0;
}

int launch_decode(Ctx* c, Op& op, const uint64_t* a) {
  DecodeShape d = shape_of(op);
  if (d.B == 0) return 0;
  const float scale = bits_f32(a[6]);
  if (!op.p0) {
    const int warps = d.B * d.H;
    TB_CUDA(c, launch_k(c, decode_generic_kernel, dim3((warps + 3) / 4), dim3(128), 0, 1, 
        (const __half*)a[0], (const __half*)a[1], (const __half*)a[2], (const int*)a[3], (const int*)a[4],
        (__half*)a[5], scale, d.B, d.H, d.G, d.D, d.NP, d.P, d.MP));
    c->launches += 1;
    TB_CUDA(c, cudaGetLastError());
    return 0;
  }
  // [NP, P, G, D] seen as (64 | D/64 * G | P | NP): a (page, kv head) tile is D/64 boxes of 16 rows x 128 bytes.
  const uint64_t key[4] = {a[1], a[2], 0, 0};
  const MapEntry* hit = op.find_maps(key);
  if (!hit) {
    const int SUB = d.D / 64;
    const uint64_t dims[4] = {64, (uint64_t)SUB * d.G, (uint64_t)d.P, (uint64_t)d.NP};
    const uint64_t strides[3] = {128, (uint64_t)d.G * d.D * 2, (uint64_t)d.P * d.G * d.D * 2};
    const uint32_t box[4] = {64, 1, 16, 1};
    CUtensorMap k4, v4;
    if (make_tensor_map(c, &k4, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, (const void*)a[1], dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B))
      return 1;
    if (make_tensor_map(c, &v4, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, (const void*)a[2], dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B))
      return 1;
    MapEntry* e = op.fresh_maps(key);
    e->m[0] = k4, e->m[1] = v4;
    hit = e;
  }
  const CUtensorMap &mk = hit->m[0], &mv = hit->m[1];
  DecodeParams p;
  p.Q = (const __half*)a[0];
  p.table = (const int*)a[3];
  p.lens = (const int*)a[4];
  p.O = (__half*)a[5];
  p.scale = scale;
  p.B = d.B;
  p.H = d.H;
  p.G = d.G;
  p.NP = d.NP;
  p.MP = d.MP;
  p.chunk = op.p1;
  p.nsplit = op.p2;
  p.part_acc = (float*)op.scratch;
  p.part_ml = p.part_acc + (size_t)d.B * d.H * p.nsplit * d.D;
  p.status = c->status;
  const int hgroups = (d.H / d.G + 7) / 8;
  dim3 grid(p.nsplit, d.G * hgroups, d.B);
  if (d.D == 128)
    TB_CUDA(c, launch_k(c, decode_tma_kernel<128>, dim3(grid), dim3(DEC_THREADS), DecSmem<128>::TOTAL, 1, mk, mv, p));
  else
    TB_CUDA(c, launch_k(c, decode_tma_kernel<64>, dim3(grid), dim3(DEC_THREADS), DecSmem<64>::TOTAL, 1, mk, mv, p));
  TB_CUDA(c, cudaGetLastError());
  c->launches += 1;
  if (p.nsplit > 1) {
    // (Merging in the first kernel, by the split that arrives last, was measured: 3-5 us slower
    // per launch at the shapes that split, because every CTA pays the fence and the count.)
    TB_CUDA(c, launch_k(c, decode_combine_kernel, dim3((d.B * d.H + 7) / 8), dim3(256), 0, 1, p, d.D, d.P));
    TB_CUDA(c, cudaGetLastError());
    c->launches += 1;
  }
  return 0;
}

}  // namespace tb

// ---------------------------------------------------------------------------------------------
// Decode attention for hosts that must not allocate device memory.
//
// tb200_kernel("decode_attention", ...) sizes and cudaMallocs the split-KV scratch when the op is
// made. Some callers cannot do that: a serving process whose whole device-memory budget was
// handed to its own pool at start-up (so any later cudaMalloc fails or fragments it), code that
// runs inside a region where the allocator must not be entered (a captured stream, a real-time
// thread), or a host that is simply forbidden to allocate after initialisation. For them the
// scratch below lives in the library image itself: every GPU that loads the library holds these
// 16 MiB until the process exits, and this entry point uses them instead of an allocation.
// ---------------------------------------------------------------------------------------------
#define TB200_STATIC_SCRATCH_BYTES (16u << 20)
static __device__ __align__(256) unsigned char g_decode_static_scratch[TB200_STATIC_SCRATCH_BYTES];

namespace tb {
namespace {
constexpr int MAX_DEVICES = 64;
// Device address of g_decode_static_scratch on each device, resolved on the first call there.
float* g_static_scratch_addr[MAX_DEVICES] = {};
}  // namespace
}  // namespace tb

struct tb200_ctx {
  tb::Ctx c;
};

extern "C" int tb200_decode_attention_static(tb200_ctx* h, const int32_t* dims, uint64_t q, uint64_t kc, uint64_t vc,
                                             uint64_t table, uint64_t lens, uint64_t o, float scale) {
  using namespace tb;
  Ctx* c = &h->c;
  if (!dims) return fail(c, "tb200_decode_attention_static: dims is NULL");
  DecodeShape d;
  d.B = dims[0], d.H = dims[1], d.G = dims[2], d.D = dims[3], d.NP = dims[4], d.P = dims[5], d.MP = dims[6];
  if (d.B < 0 || d.H < 1 || d.G < 1 || d.H % d.G || d.NP < 0 || d.P < 1 || d.MP < 0)
    return fail(c, "tb200_decode_attention_static: dims are B, H, G, D, NP, P, MP with H a multiple of G");
  if (d.D % 8 || d.D < 8 || d.D > 256)
    return fail(c, "tb200_decode_attention_static: head_dim must be a multiple of 8, at most 256");
  if (d.B == 0) return 0;
  const bool fast = d.P == 16 && (d.D == 64 || d.D == 128) && d.NP > 0 && d.MP > 0;
  if (!fast) {
    // The one-warp-per-head kernel keeps everything in registers: it has no scratch at all.
    const int warps = d.B * d.H;
    TB_CUDA(c, launch_k(c, decode_generic_kernel, dim3((warps + 3) / 4), dim3(128), 0, 1, (const __half*)q, (const __half*)kc,
                                                                  (const __half*)vc, (const int*)table,
                                                                  (const int*)lens, (__half*)o, scale, d.B, d.H, d.G,
                                                                  d.D, d.NP, d.P, d.MP));
    TB_CUDA(c, cudaGetLastError());
    c->launches += 1;
    return 0;
  }
  if (c->device < 0 || c->device >= MAX_DEVICES) return fail(c, "tb200_decode_attention_static: device index too large");
  // Set-up, once per device, with that device current. The array's name is only a host-side
  // handle for the symbol; the address a kernel may use comes from cudaGetSymbolAddress.
  TB_CUDA(c, cudaSetDevice(c->device));
  if (!g_static_scratch_addr[c->device]) {
    void* ptr = nullptr;
    TB_CUDA(c, cudaGetSymbolAddress(&ptr, g_decode_static_scratch));
    if (!ptr) return fail(c, "tb200_decode_attention_static: the scratch symbol has no device address");
    TB_CUDA(c, cudaFuncSetAttribute(decode_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    DecSmem<128>::TOTAL));
    TB_CUDA(c, cudaFuncSetAttribute(decode_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    DecSmem<64>::TOTAL));
    g_static_scratch_addr[c->device] = (float*)ptr;
  }
  // As many KV splits as the scratch can hold partials for, up to what fills the SMs.
  const size_t per_split = (size_t)d.B * d.H * (d.D + 2) * sizeof(float);
  if (per_split > TB200_STATIC_SCRATCH_BYTES) {
    char msg[256];
    snprintf(msg, sizeof msg,
             "tb200_decode_attention_static: B*H*(D+2)*4 = %zu bytes of partials exceed the %u-byte static scratch "
             "(B %d, H %d, D %d); use tb200_kernel(\"decode_attention\") instead",
             per_split, TB200_STATIC_SCRATCH_BYTES, d.B, d.H, d.D);
    return fail(c, msg);
  }
  const int hgroups = (d.H / d.G + 7) / 8;
  const long long units = (long long)d.B * d.G * hgroups;
  long long want = (4LL * c->sm_count + units - 1) / units;
  const long long fit = (long long)(TB200_STATIC_SCRATCH_BYTES / per_split);
  const int max_split = (d.MP + 3) / 4;
  if (want > fit) want = fit;
  int nsplit = (int)(want < 1 ? 1 : (want > max_split ? max_split : want));
  int chunk = (d.MP + nsplit - 1) / nsplit;
  chunk = (chunk + 3) / 4 * 4;
  nsplit = (d.MP + chunk - 1) / chunk;
  const int SUB = d.D / 64;
  CUtensorMap mk, mv;
  const uint64_t tdims[4] = {64, (uint64_t)SUB * d.G, (uint64_t)d.P, (uint64_t)d.NP};
  const uint64_t strides[3] = {128, (uint64_t)d.G * d.D * 2, (uint64_t)d.P * d.G * d.D * 2};
  const uint32_t box[4] = {64, 1, 16, 1};
  if (make_tensor_map(c, &mk, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, (const void*)kc, tdims, strides, box,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return 1;
  if (make_tensor_map(c, &mv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, (const void*)vc, tdims, strides, box,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return 1;
  DecodeParams p;
  p.Q = (const __half*)q;
  p.table = (const int*)table;
  p.lens = (const int*)lens;
  p.O = (__half*)o;
  p.scale = scale;
  p.B = d.B, p.H = d.H, p.G = d.G, p.NP = d.NP, p.MP = d.MP;
  p.chunk = chunk;
  p.nsplit = nsplit;
  // Nothing in the scratch has to start at zero: every partial the merge reads was written by
  // this call's first kernel (the merge derives the live splits from lens, as the writers do).
  p.part_acc = g_static_scratch_addr[c->device];
  p.part_ml = p.part_acc + (size_t)d.B * d.H * nsplit * d.D;
  p.status = c->status;
  dim3 grid(nsplit, d.G * hgroups, d.B);
  if (d.D == 128)
    TB_CUDA(c, launch_k(c, decode_tma_kernel<128>, dim3(grid), dim3(DEC_THREADS), DecSmem<128>::TOTAL, 1, mk, mv, p));
  else
    TB_CUDA(c, launch_k(c, decode_tma_kernel<64>, dim3(grid), dim3(DEC_THREADS), DecSmem<64>::TOTAL, 1, mk, mv, p));
  TB_CUDA(c, cudaGetLastError());
  c->launches += 1;
  if (nsplit > 1) {
    TB_CUDA(c, launch_k(c, decode_combine_kernel, dim3((d.B * d.H + 7) / 8), dim3(256), 0, 1, p, d.D, d.P));
    TB_CUDA(c, cudaGetLastError());
    c->launches += 1;
  }
  return 0;
}

