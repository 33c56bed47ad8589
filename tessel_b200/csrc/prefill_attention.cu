// Causal FlashAttention over the tokens of a step:
//   prefill_attention  packed GQA, Q/O [S,H,D], K/V [S,G,D], per-row `starts`
//                      (kernels/llm.tl:116-145)
//   flash_attention    Q/K/V/O [H,S,D]            (kernels/attention.tl:4-24)
//   chunk_attention    the next rows of a prompt that is fed in pieces, against the PAGED cache:
//                      Q/O [T,H,D], Kc/Vc [NP,16,G,D], block tables, one descriptor per chunk
//                      (no counterpart: the reference needs a prompt to fit one step,
//                      src/llm/sched.rs:76-81)
//
// tcgen05 path (D in {64, 128}): one CTA owns 256 query rows of one head as two 128-row tiles.
// A producer warp brings both Q tiles once and then 128-key K and V tiles, in the order K0 V0
// K1 V1 ..., through one ring of TMA slots. Keys are processed 64 at a time ("sub-blocks"): one
// thread issues S_t(n) = Q_t K(n)^T (M 128, N 64) into one of the tile's two 64-column score
// buffers in tensor memory, and O_t += P_t(n) V(n) (M 128, N D, K 64) with P read straight from
// tensor memory and O accumulated there. The two buffers let S_t(n+1) be computed while the
// tile's softmax warpgroup (one query row per thread) is still working on sub-block n: it reads
// S out of tensor memory, applies scale and the causal / sequence-start mask, rounds P to f16
// (as kernels/llm.tl:143 does) and stores it over the first columns of the same buffer, which
// S_t(n+2) overwrites only behind P_t(n) V(n) on the tensor pipe. So the softmax warps never
// wait for the tensor pipe in the steady state, and the two tiles fill each other's gaps. The
// running maximum is lazy: O (in tensor memory) is rescaled only when a row's maximum grew by
// more than 2^8, which leaves P <= 256 and changes no result beyond rounding; the final
// division by the row sum is exact in the same reference maximum.
//
// The key loop starts at starts[first row of the block] (not tile aligned) and
// the running maximum starts at -1e30, as the reference's does.
//
// chunk_attention runs the same pipeline with two changes: the query rows are rows
// [row0, row0 + nrows) of the step, at positions pos0, pos0 + 1, ... of their sequence, and the
// keys are positions 0 ... of that sequence read from the cache pages its block table names
// (this step's own keys were written there before the attention runs): the producer warp walks
// the table and brings each 128-key tile as eight page boxes through the 4-D tensor map the
// decode kernel uses. The causal mask compares positions.
//
// Generic path (any D that is a multiple of 8): one warp per (row, head).
#include "common.cuh"

namespace tb {

namespace {

constexpr int FA_BM = 128;        // query rows per tile (one MMA's M)
constexpr int FA_TILES = 2;       // query tiles per CTA: two softmax warpgroups take turns on the tensor pipe
constexpr int FA_BN = 128;        // keys per K / V tile in shared memory
constexpr int FA_SN = 64;         // keys per sub-block: the unit of S, softmax and P V
constexpr int FA_THREADS = 128 + FA_TILES * 128;  // warp 0 TMA, warp 1 MMA, (2, 3 idle), one softmax warpgroup per tile
// The first warpgroup gives registers back, the softmax warpgroups take them (setmaxnreg).
constexpr int FA_REGS_ISSUE = 56, FA_REGS_SOFTMAX = 216;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;  // O is rescaled only when a row's maximum grew by more than 2^8

// 2^x on the special-function unit.
__device__ __forceinline__ float exp2_sfu(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA and integer pipes: floor by a round-down add of 1.5 * 2^23 (the integer lands
// in the low mantissa bits), a degree-3 polynomial for 2^frac on [0, 1) (relative error below
// 1e-4, far inside the f16 rounding P gets next), and the integer part added to the exponent
// field. The special-function unit computes 16 exponentials per clock per SM and the softmax
// of a 128 x 64 score block needs as many of its cycles as the block's two MMAs need of the
// tensor pipe, so a share of the exponentials can be taken off it. Measured on the 8 x 32-head,
// 4096-token, D = 128 case: 981 TFLOP/s with every exponential on the special-function unit, 930
// with one in four here, 864 with one in two: the softmax warps are bound by instruction issue,
// not by that unit, and the polynomial costs about ten instructions where ex2.approx costs one.
// So the default keeps them all on the special-function unit; TB200_FA_POLY=4 selects the other.
__device__ __forceinline__ float exp2_fma(float x) {
  x = fmaxf(x, -126.0f);  // masked scores (-inf) become 2^-126: zero once rounded to f16
  float r;
  asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(x), "f"(12582912.0f));
  const float fr = x - (r - 12582912.0f);
  float p = fmaf(fr, 0.0771190897f, 0.2275643945f);
  p = fmaf(p, fr, 0.6951461434f);
  p = fmaf(p, fr, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(r) << 23));
}
constexpr int FA_POLY_DEFAULT = 0;  // one pair of exponentials in this many goes to exp2_fma (0: none)
#ifdef TB200_TRACE
__device__ unsigned long long* g_fa_trace = nullptr;  // [kind][block] timestamps (ns) of CTA (0, 0); development builds only
#define FA_TRACE(kind, jb)                                                                \
  do {                                                                                    \
    if (g_fa_trace && blockIdx.x == 0 && blockIdx.y == 0 && (jb) < 64) g_fa_trace[(kind) * 64 + (jb)] = globaltimer(); \
  } while (0)
#else
#define FA_TRACE(kind, jb) \
  do {                     \
  } while (0)
#endif

struct FaParams {
  const int* starts;  // null for the plain layout
  __half* O;
  float scale;
  int S, H, G, plain;
  unsigned int* status;
  // chunk_attention: block tables [T, MP], descriptors [C, 4] = {row0, nrows, pos0, -}, pool size.
  const int* table;
  const int* meta;
  int MP, NP, paged;
};

template <int D>
struct FaSmem {
  static constexpr int SUB = D / 64;
  static constexpr int Q_TILE = FA_BM * D * 2;
  static constexpr int Q_BYTES = FA_TILES * Q_TILE;
  static constexpr int KV_BYTES = FA_BN * D * 2;  // one K (or V) tile = one ring slot
  static constexpr int OFF_KV = Q_BYTES;
  // As many slots as fit (two are pinned by the MMAs in flight, the rest is read-ahead).
  static constexpr int NSLOT = (226 * 1024 - Q_BYTES) / KV_BYTES > 8 ? 8 : (226 * 1024 - Q_BYTES) / KV_BYTES;
  static constexpr int OFF_BAR = OFF_KV + NSLOT * KV_BYTES;
  static constexpr int TOTAL = OFF_BAR + 32 * 8 + 1024;
  // Tensor memory: tile t's two score buffers at columns [128 t + 64 b, +64), b = 0, 1 (the
  // first 32 columns of a buffer are reused for P as packed f16 pairs); O of tile t at
  // [256 + D t, 256 + D t + D).
  static constexpr int TMEM_COLS = 512;
  static_assert(NSLOT >= 4, "ring too shallow");
};

template <int D, int POLY>
__global__ void __launch_bounds__(FA_THREADS, 1)
    fa_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
              const __grid_constant__ CUtensorMap mapV, const FaParams p) {
  pdl_launch();
  pdl_wait();
  using SM = FaSmem<D>;
  constexpr int SUB = SM::SUB;
  constexpr int NSLOT = SM::NSLOT;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + SM::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;           // [NSLOT]
  uint64_t* kv_empty = bars + 1 + NSLOT;  // [NSLOT]
  uint64_t* s_full = bars + 17;           // [tile][buffer]
  uint64_t* p_ready = bars + 21;          // [tile][buffer]
  uint64_t* o_done = bars + 25;           // [tile][sub-block parity]
  uint32_t* tmem_slot = (uint32_t*)(bars + 29);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Late row blocks see the most keys: they are scheduled first so the grid's tail is short.
  const int i0 = (gridDim.x - 1 - blockIdx.x) * (FA_TILES * FA_BM), h = blockIdx.y;
  const int g = p.plain ? h : h / (p.H / p.G);
  // A row has an index in Q / O (`qrow0` + its place in the CTA) and a position among its
  // sequence's keys (`rpos0` + its place): the same number for a step's own packed keys, while a
  // chunk's rows sit at [row0, row0 + nrows) of the step and at positions pos0 ... of the cache.
  // Positions at or beyond `slim` do not exist (rows are not stored, keys are masked).
  int qrow0 = i0, rpos0 = i0, slim = p.S, trow = 0;
  if (p.paged) {
    const int* m = p.meta + 4 * blockIdx.z;
    const int row0 = m[0], nrows = m[1], pos0 = m[2];
    // A descriptor that does not lie inside the step is skipped, not trusted.
    if (row0 < 0 || nrows <= 0 || pos0 < 0 || row0 + nrows > p.S) return;
    if (i0 >= nrows) return;  // uniform for the CTA, before any barrier or tensor memory exists
    qrow0 = row0 + i0, rpos0 = pos0 + i0, slim = pos0 + nrows, trow = row0;
  }
  // Every row of the CTA starts at or after the start of its first row (prompts are packed in order).
  const int lo = p.starts ? p.starts[i0] : 0;
  // Sub-blocks of 64 keys each tile visits, counted from `lo`.
  int nsub[FA_TILES];
#pragma unroll
  for (int t = 0; t < FA_TILES; ++t) {
    const int r0 = rpos0 + t * FA_BM;
    nsub[t] = r0 < slim ? (min(r0 + FA_BM, slim) - lo + FA_SN - 1) / FA_SN : 0;
  }
  const int nmax = max(nsub[0], nsub[1]);
  const int nitems = 2 * ((nmax + 1) / 2);  // K and V tiles of 128 keys: K0 V0 K1 V1 ...

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < NSLOT; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], FA_BM);
      mbar_init(&o_done[i], 1);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, SM::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FA_REGS_ISSUE));
  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&mapQ);
      prefetch_tmap(&mapK);
      prefetch_tmap(&mapV);
      mbar_expect_tx(q_full, SM::Q_BYTES);
#pragma unroll
      for (int t = 0; t < FA_TILES; ++t)
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
          unsigned char* dst = smem + t * SM::Q_TILE + sub * (FA_BM * 128);
          if (p.plain)
            tma_load_3d(dst, &mapQ, q_full, sub * 64, qrow0 + t * FA_BM, h);
          else
            tma_load_3d(dst, &mapQ, q_full, sub * 64, h, qrow0 + t * FA_BM);
        }
    }
    int pages = 0;  // paged: lane j < 8 holds the page of keys [key0 + 16 j, key0 + 16 j + 16) of the current tile
    for (int i = 0; i < nitems; ++i) {
      const int s = i % NSLOT, k = i / NSLOT;
      const int key0 = lo + (i >> 1) * FA_BN;
      if (p.paged && (i & 1) == 0) {
        // Beyond the table, or the sequence's last page: a page outside the pool, which TMA reads as zeros.
        const int col = key0 / 16 + lane;
        pages = (lane < FA_BN / 16 && col < p.MP && col * 16 < slim) ? p.table[(size_t)trow * p.MP + col] : p.NP;
        if (pages < 0) pages = p.NP;
      }
      int page_of[FA_BN / 16];
      if (p.paged) {
#pragma unroll
        for (int j = 0; j < FA_BN / 16; ++j) page_of[j] = __shfl_sync(0xffffffffu, pages, j);
      }
      if (lane == 0) {
        const CUtensorMap* map = (i & 1) ? &mapV : &mapK;
        if (i >= NSLOT) mbar_wait(&kv_empty[s], (k & 1) ^ 1, p.status, 301);
        mbar_expect_tx(&kv_full[s], SM::KV_BYTES);
        unsigned char* dst = smem + SM::OFF_KV + s * SM::KV_BYTES;
        if (p.paged) {
#pragma unroll
          for (int j = 0; j < FA_BN / 16; ++j)
#pragma unroll
            for (int sub = 0; sub < SUB; ++sub)
              tma_load_4d(dst + sub * (FA_BN * 128) + j * 2048, map, &kv_full[s], 0, g * SUB + sub, 0, page_of[j]);
        } else {
#pragma unroll
          for (int sub = 0; sub < SUB; ++sub) {
            if (p.plain)
              tma_load_3d(dst + sub * (FA_BN * 128), map, &kv_full[s], sub * 64, key0, g);
            else
              tma_load_3d(dst + sub * (FA_BN * 128), map, &kv_full[s], sub * 64, g, key0);
          }
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_f16(FA_BM, FA_SN, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_f16(FA_BM, D, 0, 1);
      auto slot_addr = [&](int item) { return smem_u32(smem + SM::OFF_KV + (item % NSLOT) * SM::KV_BYTES); };
      // Items [0, ready) of the ring have landed.
      int ready = 0;
      auto need = [&](int item) {
        while (ready <= item) {
          mbar_wait(&kv_full[ready % NSLOT], (ready / NSLOT) & 1, p.status, 303);
          ++ready;
        }
        tc_fence_after();
      };
      // S_t(n) = Q_t K(n)^T into score buffer n & 1: keys [64 n, 64 n + 64) are rows 64 (n & 1) ...
      // of K tile n >> 1.
      auto issue_s = [&](int t, int n) {
        const uint32_t qa = smem_u32(smem + t * SM::Q_TILE);
        const uint32_t ka = slot_addr(2 * (n >> 1)) + (n & 1) * (FA_SN * 128);
#pragma unroll
        for (int kd = 0; kd < D / 16; ++kd) {
          const uint32_t off = (kd >> 2) * (FA_BM * 128) + (kd & 3) * 32;
          umma_f16(tmem + t * 128 + (n & 1) * FA_SN, umma_desc_sw128(qa + off, 16, 1024),
                   umma_desc_sw128(ka + off, 16, 1024), idesc_s, kd > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t * 2 + (n & 1)]);
      };
      // O_t (+)= P_t(n) V(n): P is read from tensor memory, V is an N-major operand in shared memory.
      auto issue_pv = [&](int t, int n) {
        const uint32_t va = slot_addr(2 * (n >> 1) + 1);
#pragma unroll
        for (int kk = 0; kk < FA_SN / 16; ++kk)
          umma_f16_ts(tmem + 256 + t * D, tmem + t * 128 + (n & 1) * FA_SN + kk * 8,
                      umma_desc_sw128(va + ((n & 1) * (FA_SN / 16) + kk) * 2048, FA_BN * 128, 1024), idesc_o,
                      (n > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&o_done[t * 2 + (n & 1)]);
      };
      mbar_wait(q_full, 0, p.status, 302);
      if (nmax > 0) {
        need(0);
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int t = 0; t < FA_TILES; ++t)
            if (n < nsub[t]) issue_s(t, n);
        umma_commit(&kv_empty[0]);  // K tile 0 is free once these are done
      }
      for (int n = 0; n < nmax; ++n) {
#pragma unroll
        for (int t = 0; t < FA_TILES; ++t) {
          if (n < nsub[t]) {
            mbar_wait(&p_ready[t * 2 + (n & 1)], (n >> 1) & 1, p.status, 304);
            FA_TRACE(8 + t, n);
            tc_fence_after();
            need(2 * (n >> 1) + 1);
            issue_pv(t, n);
          }
          if (n + 2 < nsub[t]) {
            need(2 * ((n + 2) >> 1));
            issue_s(t, n + 2);
          }
        }
        if (n & 1) {
          // Both halves of V tile n >> 1 and of K tile (n >> 1) + 1 have been issued for both tiles.
          umma_commit(&kv_empty[(n % NSLOT)]);  // item n = 2 (n >> 1) + 1
          if (n + 1 < nitems) umma_commit(&kv_empty[(n + 1) % NSLOT]);
        }
      }
    }
  } else if (warp >= 4) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FA_REGS_SOFTMAX));
    // ---- softmax: one warpgroup per tile, one query row (TMEM lane) per thread ------------------
    const int t = (warp - 4) >> 2;
    const int q = warp & 3;  // TMEM lane quadrant this warp may touch
    const int rit = q * 32 + lane;
    const int row = rpos0 + t * FA_BM + rit;  // this thread's row as a key position
    const int st = (p.starts && row < p.S) ? p.starts[row] : 0;
    const float sc2 = p.scale * LOG2E;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const uint32_t tmem_s = tmem + lane_base + t * 128;
    const uint32_t tmem_o = tmem + lane_base + 256 + t * D;
    const int nt = nsub[t];
    float m_ref = -1e30f, l = 0.f;
    for (int n = 0; n < nt; ++n) {
      const int b = n & 1;
      const int key0 = lo + n * FA_SN;
      const bool tr = t == 0 && q == 0 && lane == 0;
      if (tr) FA_TRACE(0, n);
      mbar_wait(&s_full[t * 2 + b], (n >> 1) & 1, p.status, 306);
      if (tr) FA_TRACE(1, n);
      tc_fence_after();
      uint32_t sv[FA_SN];
#pragma unroll
      for (int c = 0; c < FA_SN / 32; ++c) tmem_ld32(tmem_s + b * FA_SN + c * 32, sv + c * 32);
      tmem_ld_wait();
      if (tr) FA_TRACE(2, n);
      // Keys beyond the diagonal, before the row's own prompt, or past the end are masked.
      // Sub-blocks that lie wholly inside skip the tests. The scale (positive) is applied with
      // the subtraction of the maximum, in one fused multiply-add per score.
      const bool inside = key0 + FA_SN - 1 <= row && key0 >= st && key0 + FA_SN <= slim;
      float mx;
      if (inside) {
        // Four independent chains: one chain of dependent maxima would cost its latency 64 times.
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < FA_SN; i += 4)
#pragma unroll
          for (int u = 0; u < 4; ++u) m4[u] = fmaxf(m4[u], __uint_as_float(sv[i + u]));
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      } else {
        mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < FA_SN; ++i) {
          const int col = key0 + i;
          const bool ok = col <= row && col >= st && col < slim;
          const float x = ok ? __uint_as_float(sv[i]) : -INFINITY;
          sv[i] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      }
      mx *= sc2;  // log2 domain
      if (tr) FA_TRACE(3, n);
      const float m_new = fmaxf(m_ref, mx);
      // Lazy rescale: keep the old reference maximum unless this row outgrew it by 2^8.
      const bool grow = m_new > m_ref + RESCALE_STEP;
      if (n == 0) {
        m_ref = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        // O must be quiescent. S(n), which has completed, was issued behind P V(n-2), so only
        // P V(n-1) can still be running. Products of even and odd sub-blocks complete separate
        // barriers, so that at most one phase of a barrier is ever outstanding here and the
        // parity test is unambiguous.
        mbar_wait(&o_done[t * 2 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, p.status, 307);
        tc_fence_after();
        const float f = grow ? exp2f(m_ref - m_new) : 1.0f;
        // Eight columns at a time: the sub-block's scores stay in registers across this (rare) path.
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 8) {
          uint32_t ov[8];
          tmem_ld8(tmem_o + c0, ov);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * f);
          tmem_st8(tmem_o + c0, ov);
        }
        l *= f;
        if (grow) m_ref = m_new;
      }
      // Probabilities relative to m_ref, rounded to f16 (kernels/llm.tl:143) into tensor memory:
      // keys 2c, 2c+1 of the sub-block share column c of the buffer. The thread holds all of its
      // scores in registers, so overwriting the buffer's first columns loses nothing.
      float sum = 0.f;
      uint32_t pk[FA_SN / 2];
#pragma unroll
      for (int i = 0; i < FA_SN / 2; ++i) {
        const float xa = fmaf(__uint_as_float(sv[2 * i]), sc2, -m_ref);
        const float xb = fmaf(__uint_as_float(sv[2 * i + 1]), sc2, -m_ref);
        const bool poly = POLY > 0 && (i % (POLY > 0 ? POLY : 1)) == (POLY > 1 ? 1 : 0);
        const float a = poly ? exp2_fma(xa) : exp2_sfu(xa), b2 = poly ? exp2_fma(xb) : exp2_sfu(xb);
        sum += a + b2;
        pk[i] = pack_h2(a, b2);
      }
      if (tr) FA_TRACE(4, n);
      tmem_st32(tmem_s + b * FA_SN, pk);
      tmem_st_wait();
      if (tr) FA_TRACE(5, n);
      l += sum;
      tc_fence_before();
      mbar_arrive(&p_ready[t * 2 + b]);
    }
    if (nt > 0) {
      // The last two products may still be running (see above).
      if (nt > 1) mbar_wait(&o_done[t * 2 + ((nt - 2) & 1)], ((nt - 2) >> 1) & 1, p.status, 308);
      mbar_wait(&o_done[t * 2 + ((nt - 1) & 1)], ((nt - 1) >> 1) & 1, p.status, 309);
      tc_fence_after();
      const float inv = 1.0f / l;
      const size_t orow = (size_t)qrow0 + t * FA_BM + rit;
      __half* o = p.plain ? p.O + ((size_t)h * p.S + orow) * D : p.O + (orow * p.H + h) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t ov[32];
        tmem_ld32(tmem_o + c0, ov);
        tmem_ld_wait();
        if (row < slim) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_h2(__uint_as_float(ov[i]) * inv, __uint_as_float(ov[i + 1]) * inv);
            w.y = pack_h2(__uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv);
            w.z = pack_h2(__uint_as_float(ov[i + 4]) * inv, __uint_as_float(ov[i + 5]) * inv);
            w.w = pack_h2(__uint_as_float(ov[i + 6]) * inv, __uint_as_float(ov[i + 7]) * inv);
            *reinterpret_cast<uint4*>(o + c0 + i) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, SM::TMEM_COLS);
  }
}

// Generic path: one warp per (row, head), keys visited one at a time.
__global__ void fa_generic_kernel(const __half* __restrict__ Q, const __half* __restrict__ K,
                                  const __half* __restrict__ V, const int* __restrict__ starts, __half* __restrict__ O,
                                  float scale, int S, int H, int G, int D, int plain) {
  pdl_launch();
  pdl_wait();
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

// chunk_attention for shapes the tensor-core path does not take (any page size, any head_dim
// that is a multiple of 8): one warp per (row, head), keys visited one at a time through the
// block table; P is rounded to f16 before it weighs V, as on the tensor-core path.
__global__ void chunk_generic_kernel(const __half* __restrict__ Q, const __half* __restrict__ Kc,
                                     const __half* __restrict__ Vc, const int* __restrict__ table,
                                     const int* __restrict__ meta, __half* __restrict__ O, float scale, int T, int H,
                                     int G, int D, int NP, int P, int MP) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int* m = meta + 4 * blockIdx.y;
  const int row0 = m[0], nrows = m[1], pos0 = m[2];
  if (row0 < 0 || nrows <= 0 || pos0 < 0 || row0 + nrows > T) return;  // a descriptor outside the step is skipped
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (w >= (long long)nrows * H) return;
  const int r = (int)(w / H), h = (int)(w % H), g = h / (H / G);
  const int row = row0 + r, n = pos0 + r + 1;
  if (row >= T) return;
  constexpr int MAXC = 8;
  float q[MAXC], acc[MAXC];
  for (int c = 0; c < MAXC; ++c) {
    const int d = lane + 32 * c;
    q[c] = d < D ? __half2float(Q[((size_t)row * H + h) * D + d]) : 0.f;
    acc[c] = 0.f;
  }
  float mx = -1e30f, l = 0.f;
  for (int t = 0; t < n; ++t) {
    const int col = t / P;
    const int page = col < MP ? table[(size_t)row0 * MP + col] : 0;
    const bool in = page >= 0 && page < NP;
    const size_t at = (((size_t)(in ? page : 0) * P + t % P) * G + g) * D;
    float s = 0.f;
    for (int c = 0; c < MAXC; ++c) {
      const int d = lane + 32 * c;
      if (d < D && in) s += q[c] * __half2float(Kc[at + d]);
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    s *= scale;
    const float m2 = fmaxf(mx, s);
    const float a = expf(mx - m2), pr = expf(s - m2);
    const float p16 = __half2float(__float2half_rn(pr));
    l = l * a + pr;
    for (int c = 0; c < MAXC; ++c) {
      const int d = lane + 32 * c;
      if (d < D) acc[c] = acc[c] * a + (in ? p16 * __half2float(Vc[at + d]) : 0.f);
    }
    mx = m2;
  }
  for (int c = 0; c < MAXC; ++c) {
    const int d = lane + 32 * c;
    if (d < D) O[((size_t)row * H + h) * D + d] = __float2half_rn(acc[c] / l);
  }
}

struct FaShape {
  int S, H, G, D, plain;
  int paged = 0, NP = 0, P = 0, MP = 0, C = 0;  // chunk_attention: pool pages, page size, table width, chunks
};

FaShape fa_shape(const Op& op) {
  const auto& s = op.shapes;
  FaShape f;
  f.plain = op.kind == K_FLASH_ATTENTION;
  if (op.kind == K_CHUNK_ATTENTION) {
    // Q[T,H,D], Kc[NP,P,G,D], Vc, table[T,MP], meta[C,4], O[T,H,D]
    f.paged = 1;
    f.S = (int)s[0][0];
    f.H = (int)s[0][1];
    f.D = (int)s[0][2];
    f.NP = (int)s[1][0];
    f.P = (int)s[1][1];
    f.G = (int)s[1][2];
    f.MP = (int)s[3][1];
    f.C = (int)s[4][0];
    return f;
  }
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

template <int D, int POLY>
int run_fa(Ctx* c, Op& op, const FaShape& f, const void* Q, const void* K, const void* V, const int* starts, void* O,
           float scale, const int* table = nullptr, const int* meta = nullptr) {
  const uint64_t key[4] = {(uint64_t)Q, (uint64_t)K, (uint64_t)V, 0};
  const MapEntry* hit = op.find_maps(key);
  CUtensorMap mq, mk, mv;
  auto mk_map = [&](CUtensorMap* m, const void* base, int heads) {
    if (f.paged && base != Q) {
      // The cache [NP, 16, G, D] as the decode kernel sees it: (64 | D/64 * G | 16 | NP), one box =
      // 16 tokens x 128 bytes of one (page, kv head, 64-column block).
      const uint64_t dims[4] = {64, (uint64_t)(D / 64) * f.G, 16, (uint64_t)f.NP};
      const uint64_t strides[3] = {128, (uint64_t)f.G * D * 2, (uint64_t)16 * f.G * D * 2};
      const uint32_t box[4] = {64, 1, 16, 1};
      return make_tensor_map(c, m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, base, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    }
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
  if (hit) {
    mq = hit->m[0], mk = hit->m[1], mv = hit->m[2];
  } else {
    if (mk_map(&mq, Q, f.H) || mk_map(&mk, K, f.G) || mk_map(&mv, V, f.G)) return 1;
    MapEntry* e = op.fresh_maps(key);
    e->m[0] = mq, e->m[1] = mk, e->m[2] = mv;
  }
  FaParams p;
  p.starts = starts;
  p.O = (__half*)O;
  p.scale = scale;
  p.S = f.S;
  p.H = f.H;
  p.G = f.G;
  p.plain = f.plain;
  p.status = c->status;
  p.table = table;
  p.meta = meta;
  p.MP = f.MP;
  p.NP = f.NP;
  p.paged = f.paged;
  // chunk_attention: a chunk has at most T rows; CTAs beyond a chunk's rows leave at once.
  dim3 grid((f.S + FA_TILES * FA_BM - 1) / (FA_TILES * FA_BM), f.H, f.paged ? f.C : 1);
  TB_CUDA(c, launch_k(c, fa_kernel<D, POLY>, dim3(grid), dim3(FA_THREADS), FaSmem<D>::TOTAL, 1, mq, mk, mv, p));
  TB_CUDA(c, cudaGetLastError());
  return 0;
}

}  // namespace

int make_prefill(Ctx* c, Op& op) {
  const auto& s = op.shapes;
  auto bad = [&](const char* why) { return fail(c, op.name + ": " + why); };
  if (op.kind == K_FLASH_ATTENTION) {
    if (s[0].size() != 3 || s[1] != s[0] || s[2] != s[0] || s[3] != s[0]) return bad("shapes are Q,K,V,O [H,S,D]");
  } else if (op.kind == K_CHUNK_ATTENTION) {
    if (s[0].size() != 3 || s[1].size() != 4 || s[2] != s[1] || s[3].size() != 2 || s[4].size() != 2 || s[5] != s[0] ||
        s[3][0] != s[0][0] || s[4][1] != 4 || s[1][3] != s[0][2])
      return bad("shapes are Q[T,H,D], Kc[NP,P,G,D], Vc[NP,P,G,D], table[T,MP], meta[C,4], O[T,H,D]");
  } else {
    if (s[0].size() != 3 || s[1].size() != 3 || s[2] != s[1] || s[4] != s[0] || s[3].size() != 1 ||
        s[3][0] != s[0][0] || s[1][0] != s[0][0] || s[1][2] != s[0][2])
      return bad("shapes are Q[S,H,D], K[S,G,D], V[S,G,D], starts[S], O[S,H,D]");
  }
  const FaShape f = fa_shape(op);
  if (f.G < 1 || f.H % f.G) return bad("heads must be a multiple of kv heads");
  if (f.D % 8 || f.D > 256) return bad("head_dim must be a multiple of 8, at most 256");
  op.p0 = (f.D == 64 || f.D == 128) && f.S > 0 ? 1 : 0;
  if (f.paged && (f.P != 16 || f.NP < 1 || f.MP < 1)) op.p0 = 0;  // the page boxes are 16 tokens tall
  // TB200_FA_POLY = 0 or 4 (tuning): the share of exponentials computed off the special-function unit.
  op.p1 = FA_POLY_DEFAULT;
  if (const char* e = getenv("TB200_FA_POLY")) {
    op.p1 = atoi(e);
    if (op.p1 != 0 && op.p1 != 4) return bad("TB200_FA_POLY is 0 or 4");
  }
  if (op.p0) {
#define TB_FA_ATTR(D_, P_) \
  TB_CUDA(c, cudaFuncSetAttribute(fa_kernel<D_, P_>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaSmem<D_>::TOTAL))
    if (f.D == 128) {
      if (op.p1 == 0) TB_FA_ATTR(128, 0);
      else TB_FA_ATTR(128, 4);
    } else {
      if (op.p1 == 0) TB_FA_ATTR(64, 0);
      else TB_FA_ATTR(64, 4);
    }
#undef TB_FA_ATTR
  }
  return 0;
}

int launch_prefill(Ctx* c, Op& op, const uint64_t* a) {
  const FaShape f = fa_shape(op);
  if (f.S == 0 || f.H == 0) return 0;
  if (f.paged) {
    // Arguments: Q, Kc, Vc, table, meta, O, scale.
    if (f.C == 0) return 0;
    const void *Q = (const void*)a[0], *K = (const void*)a[1], *V = (const void*)a[2];
    const int *table = (const int*)a[3], *meta = (const int*)a[4];
    void* O = (void*)a[5];
    const float scale = bits_f32(a[6]);
    int r;
    if (op.p0) {
      if (f.D == 128)
        r = op.p1 == 0 ? run_fa<128, 0>(c, op, f, Q, K, V, nullptr, O, scale, table, meta) : run_fa<128, 4>(c, op, f, Q, K, V, nullptr, O, scale, table, meta);
      else
        r = op.p1 == 0 ? run_fa<64, 0>(c, op, f, Q, K, V, nullptr, O, scale, table, meta) : run_fa<64, 4>(c, op, f, Q, K, V, nullptr, O, scale, table, meta);
    } else {
      const long long warps = (long long)f.S * f.H;  // at most T rows per chunk
      TB_CUDA(c, launch_k(c, chunk_generic_kernel, dim3((unsigned)((warps + 3) / 4), f.C), dim3(128), 0, 1,
                          (const __half*)Q, (const __half*)K, (const __half*)V, table, meta, (__half*)O, scale, f.S, f.H,
                          f.G, f.D, f.NP, f.P, f.MP));
      cudaError_t e = cudaGetLastError();
      r = e == cudaSuccess ? 0 : cuda_fail(c, e, "chunk_generic_kernel");
    }
    if (r) return r;
    c->launches += 1;
    return 0;
  }
  const void *Q = (const void*)a[0], *K = (const void*)a[1], *V = (const void*)a[2];
  const int* starts = f.plain ? nullptr : (const int*)a[3];
  void* O = (void*)a[f.plain ? 3 : 4];
  const float scale = bits_f32(a[f.plain ? 4 : 5]);
  int r;
  if (op.p0) {
    if (f.D == 128)
      r = op.p1 == 0 ? run_fa<128, 0>(c, op, f, Q, K, V, starts, O, scale) : run_fa<128, 4>(c, op, f, Q, K, V, starts, O, scale);
    else
      r = op.p1 == 0 ? run_fa<64, 0>(c, op, f, Q, K, V, starts, O, scale) : run_fa<64, 4>(c, op, f, Q, K, V, starts, O, scale);
  } else {
    const long long warps = (long long)f.S * f.H;
    TB_CUDA(c, launch_k(c, fa_generic_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, 1, (const __half*)Q, (const __half*)K,
                                                                          (const __half*)V, starts, (__half*)O, scale,
                                                                          f.S, f.H, f.G, f.D, f.plain));
    cudaError_t e = cudaGetLastError();
    r = e == cudaSuccess ? 0 : cuda_fail(c, e, "fa_generic_kernel");
  }
  if (r) return r;
  c->launches += 1;
  return 0;
}

}  // namespace tb
