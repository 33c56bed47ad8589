// The projections of a decoder step on tcgen05 tensor cores:
//   linear           Y f16 = X W^T            kernels/llm.tl:28-36
//   linear_residual  R f32 += X W^T           kernels/llm.tl:39-47
//   logits           Y f32 = X W^T            kernels/llm.tl:50-58
//   gate_up          Y f16 = silu(X Wg^T) * (X Wu^T)   kernels/llm.tl:62-73
//   matmul           C f16 = A B, B [K,N] row-major    kernels/matmul.tl:3-17
//   linear_f32       Y f32 = X W^T (a tensor-parallel partial; no counterpart)
//   linear_scatter   linear_f32 whose rows go to their owner ranks' memory (no counterpart)
//   linear_q8, linear_residual_q8, gate_up_q8   the same three with E4M3 operands and per-row
//                    f32 scales (tcgen05 kind::f8f6f4, f32 accumulation; a non-parity mode)
//   linear_rope_kv   the QKV projection with rope_q and kv_write (kernels/llm.tl:78-112) as its
//                    epilogue: the rounded product is rotated and scattered into Q, the dense K and
//                    V and the cache pages straight from the accumulators (no counterpart as one
//                    kernel: the reference launches the three, src/llm/engine.rs:473-488)
//
// One CTA computes a (MT x 128) x BN tile of the output, MT in {1, 2}. Warp 0
// streams 64-wide K slices of both operands into a shared-memory ring with TMA
// (128-byte swizzle); one thread of warp 1 issues tcgen05.mma (M = 128, N = BN
// or 2 BN, K = 16, f16 in, f32 accumulate) into tensor memory - with MT = 2 two
// accumulators share every weight tile - and releases ring slots with
// tcgen05.commit; warps 2-9 read the finished accumulators out of tensor memory
// (one row per thread, two warps per lane quadrant taking half the columns
// each) and apply the epilogue. gate_up loads the Wg and Wu
// tiles side by side so that one MMA of N = 2 BN produces both products from
// one read of X. Rows beyond M and columns beyond N are zero-filled by TMA on
// the way in and masked on the way out.
//
// An SM takes in about 75-100 GB/s through TMA, activation and weight tiles
// together, so tiles are as large as the shape allows: a decode step's 256
// rows are ONE CTA's rows, each weight tile is fetched by one CTA only.
// Every kernel waits for its predecessor (programmatic dependent launch) only
// after it has requested its first weight tiles, which no kernel writes. Projections with few column tiles (QKV, o_proj,
// down_proj at decode sizes) would then leave SMs idle, so they split K over a
// thread-block cluster: each CTA accumulates a K range, the partial tiles are
// exchanged through distributed shared memory (every CTA owns a share of the
// tile's 128 x 32 units, the others store their partials of those units into
// its shared memory), and the owner adds them in rank order - a fixed order,
// so results do not depend on timing - before the epilogue.
//
// Shapes whose row pitch is not a multiple of 16 bytes (which TMA cannot
// address) take a plain tiled CUDA-core kernel with the same epilogues.
#include <algorithm>

#include "common.cuh"

namespace tb {

namespace {

enum Epi : int { EPI_F16 = 0, EPI_RESID = 1, EPI_F32 = 2, EPI_GATE_UP = 3, EPI_ROPE = 4 };

constexpr int BM = 128, BK = 64;
constexpr int GEMM_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue (two per TMEM lane quadrant)
constexpr int UNIT_BYTES = 128 * 32 * 4;  // one 128-row x 32-column f32 unit of a partial tile
constexpr int PAIR = 3;                   // plan code of the CTA-pair kernel (where MT is 1 or 2 otherwise)
constexpr int SCATTER_STAGE_BYTES = 8 * 4096;  // linear_scatter: 4 KB per epilogue warp, at the end of the ring

#ifdef TB200_TRACE
__device__ unsigned long long* g_trace = nullptr;  // [CTA][16] timestamps (ns), development builds only
#define TB_TRACE(point)                                                                              \
  do {                                                                                               \
    if (g_trace)                                                                                     \
      g_trace[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (point)] = globaltimer(); \
  } while (0)
#else
#define TB_TRACE(point) \
  do {                  \
  } while (0)
#endif

struct GemmParams {
  void* out;
  int M, N, K, splits;
  unsigned int* status;
  RopeArgs rope;
  // FP8 mode: f32 scales of the E4M3 operands, one per row of X and per row of W (and of Wu).
  const float *sa, *sb, *sb2;
  // linear_scatter: row r goes to rank r % n's inbox `which`, at [this rank][r / n]; null otherwise.
  const TpTable* scatter;
  int which;
};

// Where output row `row` of an f32 product starts: in `out`, or (linear_scatter) in the inbox of
// the rank that owns the row. The table is a few cache lines every thread of the grid reads.
__device__ __forceinline__ float* f32_row(const GemmParams& p, int row) {
  if (p.scatter == nullptr) return (float*)p.out + (size_t)row * p.N;
  const int n = p.scatter->nranks, src = p.scatter->rank;
  const int per = (p.M + n - 1) / n;
  return p.scatter->part[p.which][row % n] + ((size_t)src * per + row / n) * p.N;
}

template <int MT, int BN, int EPI>
struct GemmCfg {
  static constexpr int NB = EPI == EPI_GATE_UP ? 2 * BN : BN;  // B rows per stage = MMA N
  static constexpr int A_BYTES = MT * BM * BK * 2;
  static constexpr int B_BYTES = NB * BK * 2;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = (196 * 1024) / STAGE > 8 ? 8 : (196 * 1024) / STAGE;
  static constexpr int COLS = MT * NB;
  static constexpr int TMEM_COLS = COLS <= 32 ? 32 : COLS <= 64 ? 64 : COLS <= 128 ? 128 : COLS <= 256 ? 256 : 512;
  static constexpr int BAR_OFF = STAGES * STAGE;
  static constexpr int SMEM = BAR_OFF + (2 * STAGES + 1) * 8 + 16 + 1024;
  static_assert(NB % 16 == 0 && NB <= 256 && COLS <= 512, "UMMA N / TMEM columns");
  static_assert(BN % 32 == 0 || EPI == EPI_GATE_UP, "only gate_up has a ragged last chunk");
  static_assert(STAGES >= 2, "ring too shallow");
};

// linear_scatter: 32 columns of 32 rows (one per lane) into the owner ranks' inboxes. A thread
// holds a row, and a row's owner is another GPU more often than not: storing straight from the
// registers would cross NVLink as 16-byte pieces of 32 different rows per instruction, which
// measured 17 us on top of a 22 us projection. So the warp turns the 32 x 32 block round in 4 KB
// of shared memory (chunks XOR-swizzled by row: no bank conflicts either way) and stores row by
// row, 128 contiguous bytes per instruction.
__device__ __forceinline__ void scatter_store(const GemmParams& p, float* stage, int row, int col0, const float* v) {
  const int lane = threadIdx.x & 31;
  float4* sw = reinterpret_cast<float4*>(stage);
#pragma unroll
  for (int j = 0; j < 8; ++j) sw[lane * 8 + (j ^ (lane & 7))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  __syncwarp();
  const int row0 = row - lane;
  const bool col_ok = col0 + lane < p.N;
  // Consecutive rows go round the owners: no division per row.
  const TpTable* t = p.scatter;
  const int n = t->nranks, per = (p.M + n - 1) / n;
  int owner = row0 % n;
  size_t at = ((size_t)t->rank * per + row0 / n) * p.N + col0 + lane;  // offset in the owner's inbox
  float* const* inbox = t->part[p.which];
#pragma unroll 4
  for (int r = 0; r < 32; ++r) {
    float val = stage[r * 32 + (((lane >> 2) ^ (r & 7)) << 2) + (lane & 3)];
    // 0xffffffff marks an empty inbox word (csrc/tp.cu): that NaN goes out as another NaN.
    if (__float_as_uint(val) == 0xffffffffu) val = __uint_as_float(0x7fffffffu);
    if (row0 + r < p.M && col_ok) inbox[owner][at] = val;
    if (++owner == n) {
      owner = 0;
      at += p.N;
    }
  }
  __syncwarp();
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  // g / (1 + exp(-g)) * u (kernels/llm.tl:73) on the fast exponential and division units:
  // a few f32 ulps from the interpreter's op-by-op rounding, far inside the f16 output step.
#ifdef TB200_EXACT_SILU
  const float e = expf(-g);
  return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, e)), u);
#else
  return __fdividef(g, 1.0f + __expf(-g)) * u;
#endif
}

// Writes up to 32 consecutive columns of one output row (col0 .. col0 + ncols - 1, clipped to N).
template <int EPI>
__device__ __forceinline__ void store_chunk(const GemmParams& p, int row, int col0, const float* v, int ncols = 32) {
  if (row >= p.M || col0 >= p.N) return;
  const bool fullw = ncols == 32 && col0 + 32 <= p.N && (p.N % 8) == 0;
  if (EPI == EPI_F16 || EPI == EPI_GATE_UP) {
    __half* y = (__half*)p.out + (size_t)row * p.N + col0;
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
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols && col0 + j < p.N) y[j] = __float2half_rn(v[j]);
    }
  } else {
    float* y = (EPI == EPI_F32 ? f32_row(p, row) : (float*)p.out + (size_t)row * p.N) + col0;
    if (fullw) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
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
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols && col0 + j < p.N) y[j] = EPI == EPI_RESID ? __fadd_rn(y[j], v[j]) : v[j];
    }
  }
}

// One rotated pair (kernels/llm.tl:85-88): products and sums rounded separately, as the
// interpreter does, so that the pages written from here are the reference's bits.
__device__ __forceinline__ void rope_pair(float x1, float x2, float c, float s, float& y1, float& y2) {
  y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
  y2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
}

__device__ __forceinline__ void store_h32(__half* dst, const float* v) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 o;
    o.x = pack_h2(v[j], v[j + 1]);
    o.y = pack_h2(v[j + 2], v[j + 3]);
    o.z = pack_h2(v[j + 4], v[j + 5]);
    o.w = pack_h2(v[j + 6], v[j + 7]);
    *reinterpret_cast<uint4*>(dst + j) = o;
  }
}

// linear_rope_kv: 32 columns of each half of one head of one row. `v1` holds columns
// [32 hu, 32 hu + 32) of the head that starts at column `gc` of QKV, `v2` the same columns of
// the head's second half. The product is rounded to f16 first (the reference's qkv buffer is
// f16), stored to QKV, and then: a query head is rotated into Q; a key head is rotated into the
// dense K and, unless the row's slot is outside the cache, its page; a value head is copied to
// the dense V and its page.
__device__ __forceinline__ void rope_store(const GemmParams& p, int row, int gc, int hu, float* v1, float* v2) {
  const RopeArgs& a = p.rope;
  const int D = a.D, d2 = D >> 1, HD = a.H * D, GD = a.G * D;
  if (row >= p.M || gc >= p.N) return;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    v1[j] = __half2float(__float2half_rn(v1[j]));
    v2[j] = __half2float(__float2half_rn(v2[j]));
  }
  const int off = hu * 32;
  __half* qkv = (__half*)p.out + (size_t)row * p.N + gc + off;
  store_h32(qkv, v1);
  store_h32(qkv + d2, v2);
  const int at = a.slot[row];
  const bool keep = at >= 0 && at < a.NS;
  if (gc >= HD + GD) {
    const int g = (gc - HD - GD) / D;
    __half* vd = a.Vd + ((size_t)row * a.G + g) * D + off;
    store_h32(vd, v1);
    store_h32(vd + d2, v2);
    if (keep) {
      __half* vc = a.Vc + ((size_t)at * a.G + g) * D + off;
      store_h32(vc, v1);
      store_h32(vc + d2, v2);
    }
    return;
  }
  const int ps = a.pos[row];
  const bool in = ps >= 0 && ps < a.NPOS;
  const float* ct = a.Ct + (size_t)(in ? ps : 0) * d2 + off;
  const float* st = a.St + (size_t)(in ? ps : 0) * d2 + off;
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 c = in ? *reinterpret_cast<const float4*>(ct + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 sn = in ? *reinterpret_cast<const float4*>(st + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    float y1, y2;
    rope_pair(v1[j], v2[j], c.x, sn.x, y1, y2), v1[j] = y1, v2[j] = y2;
    rope_pair(v1[j + 1], v2[j + 1], c.y, sn.y, y1, y2), v1[j + 1] = y1, v2[j + 1] = y2;
    rope_pair(v1[j + 2], v2[j + 2], c.z, sn.z, y1, y2), v1[j + 2] = y1, v2[j + 2] = y2;
    rope_pair(v1[j + 3], v2[j + 3], c.w, sn.w, y1, y2), v1[j + 3] = y1, v2[j + 3] = y2;
  }
  if (gc < HD) {
    __half* q = a.Q + ((size_t)row * a.H + gc / D) * D + off;
    store_h32(q, v1);
    store_h32(q + d2, v2);
    return;
  }
  const int g = (gc - HD) / D;
  __half* kd = a.Kd + ((size_t)row * a.G + g) * D + off;
  store_h32(kd, v1);
  store_h32(kd + d2, v2);
  if (keep) {
    __half* kc = a.Kc + ((size_t)at * a.G + g) * D + off;
    store_h32(kc, v1);
    store_h32(kc + d2, v2);
  }
}

// FP8 mode: 32 accumulator columns of one row back to real units: x (row scale of X) x (row
// scale of W, one per output column).
__device__ __forceinline__ void q8_scale(const GemmParams& p, const float* sb, int row, int col0, float* v) {
  const float sa = row < p.M ? p.sa[row] : 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] *= sa * (col0 + j < p.N ? sb[col0 + j] : 0.f);
}

// The epilogue of one CTA: warps 2-9 read the CTA's MT x 128 rows of the finished accumulators
// out of tensor memory (TMEM lane quadrant = warp % 4, one output row per thread; the two warps
// of a quadrant share the 32-column units between them) and store them. With S > 1 the S CTAs
// that split K first exchange partial tiles through distributed shared memory: the tile's
// 128 x 32 units are dealt to the splits in groups (a group is one unit, or for linear_rope_kv
// the units of one head, which must meet in one CTA), every CTA stores its partial of a unit
// into the ring (idle by then) of the unit's owner, and the owner adds the partials in split
// order. `split` is this CTA's index among the S; the CTA holding split s of the same tile has
// cluster rank s * rank_stride + rank_off.
template <int MT, int BN, int NB, int EPI, bool Q8 = false>
__device__ __forceinline__ void tile_epilogue(const GemmParams& p, uint32_t tmem, unsigned char* smem,
                                              uint64_t* acc_full, int m0, int n0, int S, uint32_t split,
                                              uint32_t rank_stride, uint32_t rank_off, int ring_bytes) {
  constexpr int CH = BN / 32;
  constexpr int UNITS = MT * CH;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool epi = warp >= 2;
  const int q = warp & 3;
  const int eh = (warp - 2) >> 2;
  const uint32_t lane_base = (uint32_t)(q * 32) << 16;
  const bool tracer = warp == 2 && lane == 0;
  const int rit = q * 32 + lane;  // row within a 128-row block
  // Units that stay together (one owner): a head for linear_rope_kv (BN is a multiple of D there).
  const int UH = EPI == EPI_ROPE ? p.rope.D / 32 : 1;
  const int groups = UNITS / UH;
  const int per = ((groups + S - 1) / S) * UH;  // units each CTA owns, at most
  auto owner_of = [&](int u) { return (uint32_t)((u / UH) % S); };
  auto slot_of = [&](int u) { return ((u / UH) / S) * UH + u % UH; };
  float* recv = (float*)smem;  // [(S - 1) senders][per][8 float4 columns][128 rows]
  // linear_scatter: 4 KB per epilogue warp at the end of the ring (idle by now; the received
  // partials sit at its start), to turn blocks round before they leave for other GPUs.
  float* turn = (float*)(smem + ring_bytes - SCATTER_STAGE_BYTES) + (warp - 2) * 1024;
  const bool scatter = EPI == EPI_F32 && p.scatter != nullptr;
  if (epi) {
    pdl_wait();  // the epilogue reads and writes buffers other kernels touch
    mbar_wait(acc_full, 0, p.status, 203);
    tc_fence_after();
    if (tracer) TB_TRACE(4);
  }
  if (S > 1) {
    // Split K: exchange partial tiles through distributed shared memory.
    __syncwarp();
    cluster_sync();  // every CTA of the cluster has finished its MMAs: all rings are free
    if (tracer) TB_TRACE(5);
    if (epi) {
      for (int u = 0; u < UNITS; ++u) {
        const uint32_t owner = owner_of(u);
        if (owner == split || (u & 1) != eh) continue;
        const int mt = u / CH, c0 = (u % CH) * 32;
        uint32_t r[32];
        tmem_ld32(tmem + lane_base + mt * NB + c0, r);
        tmem_ld_wait();
        const uint32_t sidx = split < owner ? split : split - 1;  // my place among the owner's senders
        const uint32_t local = smem_u32(recv) + (sidx * per + slot_of(u)) * UNIT_BYTES + rit * 16;
        const uint32_t remote = cluster_map(local, owner * rank_stride + rank_off);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          st_cluster_f4(remote + j * 2048, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                        __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
      }
    }
    if (tracer) TB_TRACE(6);
    __syncwarp();
    cluster_sync();  // all partials have landed
    if (tracer) TB_TRACE(7);
  }
  // The 32 finished columns of unit u (owned by this CTA): the accumulator, plus, in split order
  // 0, 1, ..., S-1 whatever the timing, the partials the other splits sent.
  auto sum_unit = [&](int u, float* v) {
    const int mt = u / CH, c0 = (u % CH) * 32;
    uint32_t r[32];
    tmem_ld32(tmem + lane_base + mt * NB + c0, r);
    tmem_ld_wait();
    if (S == 1) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      return;
    }
    const int slot = slot_of(u);
    for (int s = 0; s < S; ++s) {
      if ((uint32_t)s == split) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = s == 0 ? __uint_as_float(r[j]) : __fadd_rn(v[j], __uint_as_float(r[j]));
      } else {
        const int sidx = (uint32_t)s < split ? s : s - 1;
        const float4* src = (const float4*)((const unsigned char*)recv + (sidx * per + slot) * UNIT_BYTES) + rit;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 t = src[j * 128];
          if (s == 0) {
            v[4 * j] = t.x, v[4 * j + 1] = t.y, v[4 * j + 2] = t.z, v[4 * j + 3] = t.w;
          } else {
            v[4 * j] = __fadd_rn(v[4 * j], t.x);
            v[4 * j + 1] = __fadd_rn(v[4 * j + 1], t.y);
            v[4 * j + 2] = __fadd_rn(v[4 * j + 2], t.z);
            v[4 * j + 3] = __fadd_rn(v[4 * j + 3], t.w);
          }
        }
      }
    }
  };
  if (!epi) return;
  if (EPI == EPI_ROPE) {
    // Whole heads: a thread takes columns [32 hu, 32 hu + 32) of both halves of a head at a time.
    int item = 0;
    for (int gi = (int)split; gi < groups; gi += S) {
      const int u0 = gi * UH, mt = u0 / CH, gc = n0 + (u0 % CH) * 32;
      for (int hu = 0; hu < UH / 2; ++hu, ++item) {
        if ((item & 1) != eh) continue;
        float v1[32], v2[32];
        sum_unit(u0 + hu, v1);
        sum_unit(u0 + UH / 2 + hu, v2);
        rope_store(p, m0 + mt * BM + rit, gc, hu, v1, v2);
      }
    }
    return;
  }
  if (S == 1) {
#pragma unroll 1
    for (int mt = 0; mt < MT; ++mt) {
      const int row = m0 + mt * BM + rit;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (((c0 >> 5) & 1) != eh) continue;
        uint32_t r[32];
        float v[32];
        tmem_ld32(tmem + lane_base + mt * NB + c0, r);
        if (EPI == EPI_GATE_UP) {
          uint32_t r2[32];
          tmem_ld32(tmem + lane_base + mt * NB + BN + c0, r2);
          tmem_ld_wait();
          if (Q8) {
            float u[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]), u[j] = __uint_as_float(r2[j]);
            q8_scale(p, p.sb, row, n0 + c0, v);
            q8_scale(p, p.sb2, row, n0 + c0, u);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = silu_mul(v[j], u[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = silu_mul(__uint_as_float(r[j]), __uint_as_float(r2[j]));
          }
        } else {
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (Q8) q8_scale(p, p.sb, row, n0 + c0, v);
        }
        if (scatter)
          scatter_store(p, turn, row, n0 + c0, v);
        else
          store_chunk<EPI>(p, row, n0 + c0, v, BN - c0 < 32 ? BN - c0 : 32);
      }
    }
  } else {
    int item = 0;
    for (int gi = (int)split; gi < groups; gi += S, ++item) {
      if ((item & 1) != eh) continue;
      const int u = gi;  // groups are single units here
      float v[32];
      sum_unit(u, v);
      if (Q8) q8_scale(p, p.sb, m0 + (u / CH) * BM + rit, n0 + (u % CH) * 32, v);
      if (scatter)
        scatter_store(p, turn, m0 + (u / CH) * BM + rit, n0 + (u % CH) * 32, v);
      else
        store_chunk<EPI>(p, m0 + (u / CH) * BM + rit, n0 + (u % CH) * 32, v);
    }
  }
}

// B_MN: B is a [K, N] row-major array (N-major operand); else W [N, K] (K-major).
// Grid: (row tiles, column tiles, K splits); with splits > 1 the launch carries a
// cluster of (1, 1, splits).
template <int MT, int BN, int EPI, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                const __grid_constant__ CUtensorMap mapB2, const GemmParams p) {
  using Cfg = GemmCfg<MT, BN, EPI>;
  constexpr int NB = Cfg::NB, STAGES = Cfg::STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + Cfg::BAR_OFF);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * (MT * BM), n0 = blockIdx.y * BN;
  const int nk = (p.K + BK - 1) / BK;
  const int S = p.splits;
  const int k_begin = (int)((long long)nk * blockIdx.z / S), k_end = (int)((long long)nk * (blockIdx.z + 1) / S);
  const int niter = k_end - k_begin;  // >= 1: the host never asks for more splits than K blocks

  pdl_launch();
  if (threadIdx.x == 0) {
    TB_TRACE(0);
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
      TB_TRACE(1);
      // The weights are not written by any kernel of the stream, so their first tiles are
      // fetched before waiting for the previous kernel; the activations (A) only after it.
      const int pre = B_MN ? 0 : (niter < STAGES ? niter : STAGES);
      auto load_b = [&](int i) {
        const int s = i % STAGES, kc = (k_begin + i) * BK;
        unsigned char* b = smem + s * Cfg::STAGE + Cfg::A_BYTES;
        mbar_expect_tx(&full[s], Cfg::STAGE);
        if (B_MN) {
          // 64-column blocks of [64 k-rows x 128 bytes] each.
#pragma unroll
          for (int nb = 0; nb < BN / 64; ++nb) tma_load_2d(b + nb * (BK * 128), &mapB, &full[s], n0 + nb * 64, kc);
        } else {
          tma_load_2d(b, &mapB, &full[s], kc, n0);
          if (EPI == EPI_GATE_UP) tma_load_2d(b + BN * BK * 2, &mapB2, &full[s], kc, n0);
        }
      };
      for (int i = 0; i < pre; ++i) load_b(i);
      pdl_wait();
      for (int i = 0; i < niter; ++i) {
        const int s = i % STAGES, k = i / STAGES, kc = (k_begin + i) * BK;
        if (i >= pre) {
          mbar_wait(&empty[s], (k & 1) ^ 1, p.status, 201);
          load_b(i);
        }
        tma_load_2d(smem + s * Cfg::STAGE, &mapA, &full[s], kc, m0);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16(BM, NB, 0, B_MN ? 1 : 0);
      for (int i = 0; i < niter; ++i) {
        const int s = i % STAGES, k = i / STAGES;
        mbar_wait(&full[s], k & 1, p.status, 202);
        if (i == 0) TB_TRACE(2);
        tc_fence_after();
        const uint32_t a = smem_u32(smem + s * Cfg::STAGE);
        const uint32_t b = a + Cfg::A_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          const uint64_t bd = B_MN ? umma_desc_sw128(b + kk * 2048, BK * 128, 1024)
                                   : umma_desc_sw128(b + kk * 32, 16, 1024);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint64_t ad = umma_desc_sw128(a + mt * (BM * 128) + kk * 32, 16, 1024);
            umma_f16(tmem + mt * NB, ad, bd, idesc, (i > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty[s]);  // frees the slot once these MMAs have read it
      }
      TB_TRACE(3);
      umma_commit(acc_full);
    }
  }

  tile_epilogue<MT, BN, NB, EPI>(p, tmem, smem, acc_full, m0, n0, S, S > 1 ? cluster_ctarank() : 0u, 1u, 0u, Cfg::BAR_OFF);
  const bool tracer = warp == 2 && lane == 0;
  if (tracer) TB_TRACE(8);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// ---- CTA pairs ------------------------------------------------------------------------
// With 129 to 256 rows per tile (a decode step), one CTA has to take in its whole activation
// tile again for every weight tile, and what an SM can take in through TMA is the bound: half of
// it goes to activations. A CTA PAIR (tcgen05 cta_group::2) halves that share: the two CTAs of a
// cluster run one MMA of M = 256 together, each keeping only ITS 128 rows of the activation
// slice and HALF of the weight slice's rows in its own shared memory; the even CTA issues the
// MMAs, each CTA ends up with its 128 rows of the accumulator in its own tensor memory and runs
// the same epilogue as above on them. gate_up issues two MMAs per K step (gate and up columns)
// so that a pair covers BN output columns with 2 BN accumulator columns per CTA.
template <int BN, int EPI>
struct PairCfg {
  static constexpr int NOPS = EPI == EPI_GATE_UP ? 2 : 1;  // weight matrices
  static constexpr int NBH = BN / 2;                       // rows of each weight slice this CTA loads
  static constexpr int NB = NOPS * BN;                     // accumulator columns per CTA
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = NOPS * NBH * BK * 2;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = (196 * 1024) / STAGE > 8 ? 8 : (196 * 1024) / STAGE;
  static constexpr int TMEM_COLS = NB <= 32 ? 32 : NB <= 64 ? 64 : NB <= 128 ? 128 : NB <= 256 ? 256 : 512;
  static constexpr int BAR_OFF = STAGES * STAGE;
  static constexpr int SMEM = BAR_OFF + (2 * STAGES + 1) * 8 + 16 + 1024;
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256 && NB <= 512, "UMMA N (M = 256: a multiple of 16) / TMEM columns");
  static_assert(NBH % 8 == 0 && STAGE % 1024 == 0, "swizzle atoms are 8 rows of 128 bytes");
  static_assert(STAGES >= 2, "ring too shallow");
};

// Grid: (2 x row pairs, column tiles, K splits), cluster (2, 1, splits): cluster rank =
// (blockIdx.x & 1) + 2 * split. K-major weights only (W [N, K]).
template <int BN, int EPI, bool Q8 = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                     const __grid_constant__ CUtensorMap mapB2, const GemmParams p) {
  using Cfg = PairCfg<BN, EPI>;
  constexpr int STAGES = Cfg::STAGES, NBH = Cfg::NBH;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + Cfg::BAR_OFF);  // used in the even CTA only: both CTAs' loads count there
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);

  const int warp = threadIdx.x >> 5;
  const uint32_t crank = cluster_ctarank();
  const uint32_t half = crank & 1u;        // which 128 rows of the pair's 256
  const uint32_t leader = crank & ~1u;     // cluster rank of the pair's even CTA
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  // A stage holds 128 bytes of K per row either way: 64 halves, or (FP8 mode) 128 E4M3 bytes.
  constexpr int BKE = Q8 ? 2 * BK : BK;
  const int nk = (p.K + BKE - 1) / BKE;
  const int S = p.splits;
  const int k_begin = (int)((long long)nk * blockIdx.z / S), k_end = (int)((long long)nk * (blockIdx.z + 1) / S);
  const int niter = k_end - k_begin;

  pdl_launch();
  if (threadIdx.x == 0) {
    TB_TRACE(0);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the partner's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      prefetch_tmap(&mapA);
      prefetch_tmap(&mapB);
      if (EPI == EPI_GATE_UP) prefetch_tmap(&mapB2);
      TB_TRACE(1);
      // As in gemm_kernel: weight tiles are requested before waiting for the previous kernel.
      const int pre = niter < STAGES ? niter : STAGES;
      auto load_b = [&](int i) {
        const int s = i % STAGES, kc = (k_begin + i) * BKE;
        unsigned char* b = smem + s * Cfg::STAGE + Cfg::A_BYTES;
        const uint32_t bar = cluster_map(smem_u32(&full[s]), leader);
        if (half == 0) mbar_expect_tx(&full[s], 2 * Cfg::STAGE);  // this CTA's tiles and the partner's
        tma_load_2d_pair(b, &mapB, bar, kc, n0 + (int)half * NBH);
        if (EPI == EPI_GATE_UP) tma_load_2d_pair(b + NBH * BK * 2, &mapB2, bar, kc, n0 + (int)half * NBH);
      };
      for (int i = 0; i < pre; ++i) load_b(i);
      pdl_wait();
      for (int i = 0; i < niter; ++i) {
        const int s = i % STAGES, k = i / STAGES, kc = (k_begin + i) * BKE;
        if (i >= pre) {
          mbar_wait(&empty[s], (k & 1) ^ 1, p.status, 211);
          load_b(i);
        }
        tma_load_2d_pair(smem + s * Cfg::STAGE, &mapA, cluster_map(smem_u32(&full[s]), leader), kc, m0);
      }
    }
  } else if (warp == 1 && half == 0) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16(2 * BM, BN, 0, 0);
      const uint16_t both = (uint16_t)(3u << leader);
      for (int i = 0; i < niter; ++i) {
        const int s = i % STAGES, k = i / STAGES;
        mbar_wait(&full[s], k & 1, p.status, 212);
        if (i == 0) TB_TRACE(2);
        tc_fence_after();
        const uint32_t a = smem_u32(smem + s * Cfg::STAGE);
        const uint32_t b = a + Cfg::A_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(a + kk * 32, 16, 1024);
#pragma unroll
          for (int op = 0; op < Cfg::NOPS; ++op) {
            const uint64_t bd = umma_desc_sw128(b + op * (NBH * BK * 2) + kk * 32, 16, 1024);
            if (Q8)
              umma_q8_pair(tmem + op * BN, ad, bd, idesc, (i > 0 || kk > 0) ? 1u : 0u);
            else
              umma_f16_pair(tmem + op * BN, ad, bd, idesc, (i > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit_pair(&empty[s], both);  // frees the slot in both CTAs once these MMAs have read it
      }
      TB_TRACE(3);
      umma_commit_pair(acc_full, both);
    }
  }
  __syncwarp();
  tile_epilogue<1, BN, Cfg::NB, EPI, Q8>(p, tmem, smem, acc_full, m0, n0, S, crank >> 1, 2u, half, Cfg::BAR_OFF);
  if (warp == 2 && (threadIdx.x & 31) == 0) TB_TRACE(8);
  // Both CTAs have read their accumulators (and every barrier signal of the pair has landed)
  // before either frees tensor memory or leaves.
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, Cfg::TMEM_COLS);
  }
}

// CUDA-core path for pitches TMA cannot address: 32 x 32 output tile per block.
template <int EPI, bool B_MN>
__global__ void gemm_plain_kernel(const __half* __restrict__ A, const __half* __restrict__ B,
                                  const __half* __restrict__ B2, void* __restrict__ out, int M, int N, int K) {
  pdl_launch();
  pdl_wait();
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
  int D = 0;  // linear_rope_kv: head_dim (a tile must hold whole heads)
  int q8 = 0;  // FP8 kinds: a K slice is 128 elements, CTA pairs only
};

GemmShape gemm_shape(const Op& op) {
  const auto& s = op.shapes;
  GemmShape g;
  g.M = (int)s[0][0];
  g.K = (int)s[0][1];
  g.N = op.kind == K_MATMUL ? (int)s[1][1] : (int)s[1][0];
  // FP8 kinds: Xq[M,K], sx[M], Wq[N,K], sw[N], (Wuq[N,K], su[N],) out[M,N]
  if (op.kind == K_LINEAR_Q8 || op.kind == K_LINEAR_RESIDUAL_Q8 || op.kind == K_GATE_UP_Q8) {
    g.N = (int)s[2][0];
    g.q8 = 1;
  }
  if (op.kind == K_LINEAR_ROPE_KV) g.D = (int)s[7][2];  // Q[T,H,D]
  return g;  // linear_scatter, linear_rope_kv: X[M,K], W[N,K] lead as in linear
}

int epi_of(Kind k) {
  switch (k) {
    case K_LINEAR:
    case K_MATMUL:
    case K_LINEAR_Q8:
      return EPI_F16;
    case K_LINEAR_RESIDUAL:
    case K_LINEAR_RESIDUAL_Q8:
      return EPI_RESID;
    case K_GATE_UP:
    case K_GATE_UP_Q8:
      return EPI_GATE_UP;
    case K_LINEAR_ROPE_KV:
      return EPI_ROPE;
    default:
      return EPI_F32;
  }
}

template <int MT, int BN, int EPI, bool B_MN>
int run(Ctx* c, Op& op, const GemmShape& g, int splits, const void* A, const void* B, const void* B2, void* out,
        bool attr_only) {
  using Cfg = GemmCfg<MT, BN, EPI>;
  if (attr_only) {
    TB_CUDA(c, cudaFuncSetAttribute(gemm_kernel<MT, BN, EPI, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::SMEM));
    return 0;
  }
  const uint64_t key[4] = {(uint64_t)A, (uint64_t)B, (uint64_t)B2, ((uint64_t)MT << 32) | ((uint64_t)BN << 8) | (uint64_t)splits};
  const MapEntry* hit = op.find_maps(key);
  if (!hit) {
    CUtensorMap ma, mb, mb2;
    {
      const uint64_t dims[2] = {(uint64_t)g.K, (uint64_t)g.M};
      const uint64_t strides[1] = {(uint64_t)g.K * 2};
      const uint32_t box[2] = {BK, MT * BM};
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
    MapEntry* e = op.fresh_maps(key);
    e->m[0] = ma, e->m[1] = mb, e->m[2] = mb2;
    hit = e;
  }
  const CUtensorMap &ma = hit->m[0], &mb = hit->m[1], &mb2 = hit->m[2];
  GemmParams p;
  p.out = out;
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.splits = splits;
  p.status = c->status;
  p.scatter = op.kind == K_LINEAR_SCATTER ? (const TpTable*)out : nullptr;
  p.which = op.aux;
  p.rope = op.rope;
  p.sa = p.sb = p.sb2 = nullptr;
  const dim3 grid((g.M + MT * BM - 1) / (MT * BM), (g.N + BN - 1) / BN, splits);
  TB_CUDA(c, launch_k(c, gemm_kernel<MT, BN, EPI, B_MN>, grid, dim3(GEMM_THREADS), Cfg::SMEM, splits, ma, mb, mb2, p));
  return 0;
}

template <int BN, int EPI, bool Q8 = false>
int run_pair(Ctx* c, Op& op, const GemmShape& g, int splits, const void* A, const void* B, const void* B2, void* out,
             bool attr_only) {
  using Cfg = PairCfg<BN, EPI>;
  if (attr_only) {
    TB_CUDA(c, cudaFuncSetAttribute(gemm_pair_kernel<BN, EPI, Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
    return 0;
  }
  const uint64_t key[4] = {(uint64_t)A, (uint64_t)B, (uint64_t)B2, ((uint64_t)PAIR << 32) | ((uint64_t)BN << 8) | (uint64_t)splits};
  // Rows of 128 bytes of K either way: 64 halves, or 128 E4M3 bytes.
  const CUtensorMapDataType dt = Q8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const uint64_t pitch = (uint64_t)g.K * (Q8 ? 1 : 2);
  const uint32_t bk = Q8 ? 2 * BK : BK;
  const MapEntry* hit = op.find_maps(key);
  if (!hit) {
    CUtensorMap ma, mb, mb2;
    {
      const uint64_t dims[2] = {(uint64_t)g.K, (uint64_t)g.M};
      const uint64_t strides[1] = {pitch};
      const uint32_t box[2] = {bk, BM};
      if (make_tensor_map(c, &ma, dt, 2, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
        return 1;
    }
    {
      const uint64_t dims[2] = {(uint64_t)g.K, (uint64_t)g.N};
      const uint64_t strides[1] = {pitch};
      const uint32_t box[2] = {bk, Cfg::NBH};
      if (make_tensor_map(c, &mb, dt, 2, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
        return 1;
      mb2 = mb;
      if (EPI == EPI_GATE_UP &&
          make_tensor_map(c, &mb2, dt, 2, B2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
        return 1;
    }
    MapEntry* e = op.fresh_maps(key);
    e->m[0] = ma, e->m[1] = mb, e->m[2] = mb2;
    hit = e;
  }
  const CUtensorMap &ma = hit->m[0], &mb = hit->m[1], &mb2 = hit->m[2];
  GemmParams p;
  p.out = out;
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.splits = splits;
  p.status = c->status;
  p.scatter = op.kind == K_LINEAR_SCATTER ? (const TpTable*)out : nullptr;
  p.which = op.aux;
  p.rope = op.rope;
  p.sa = op.q8[0], p.sb = op.q8[1], p.sb2 = op.q8[2];
  const dim3 grid(2 * ((g.M + 2 * BM - 1) / (2 * BM)), (g.N + BN - 1) / BN, splits);
  TB_CUDA(c, launch_kc(c, gemm_pair_kernel<BN, EPI, Q8>, grid, dim3(GEMM_THREADS), Cfg::SMEM, 2, splits, ma, mb, mb2, p));
  return 0;
}

bool is_q8(Kind k) { return k == K_LINEAR_Q8 || k == K_LINEAR_RESIDUAL_Q8 || k == K_GATE_UP_Q8; }

template <int BN>
int dispatch_pair(Ctx* c, Op& op, Kind kind, const GemmShape& g, int splits, const void* A, const void* B, const void* B2,
                  void* out, bool attr_only) {
  if (is_q8(kind)) {
    if constexpr (BN == 128 || BN == 256) {
      if (kind == K_GATE_UP_Q8) return run_pair<BN, EPI_GATE_UP, true>(c, op, g, splits, A, B, B2, out, attr_only);
      if (kind == K_LINEAR_Q8) return run_pair<BN, EPI_F16, true>(c, op, g, splits, A, B, B2, out, attr_only);
      return run_pair<BN, EPI_RESID, true>(c, op, g, splits, A, B, B2, out, attr_only);
    }
    return fail(c, "gemm: FP8 tiles are 128 or 256 columns wide");
  }
  switch (epi_of(kind)) {
    case EPI_GATE_UP:
      return run_pair<BN, EPI_GATE_UP>(c, op, g, splits, A, B, B2, out, attr_only);
    case EPI_F16:
      return run_pair<BN, EPI_F16>(c, op, g, splits, A, B, B2, out, attr_only);
    case EPI_RESID:
      return run_pair<BN, EPI_RESID>(c, op, g, splits, A, B, B2, out, attr_only);
    case EPI_ROPE:
      if constexpr (BN == 128 || BN == 256) return run_pair<BN, EPI_ROPE>(c, op, g, splits, A, B, B2, out, attr_only);
      return fail(c, "gemm: linear_rope_kv pair tiles are 128 or 256 columns wide");
    default:
      return run_pair<BN, EPI_F32>(c, op, g, splits, A, B, B2, out, attr_only);
  }
}

template <int EPI, bool B_MN>
int run_plain(Ctx* c, const GemmShape& g, const void* A, const void* B, const void* B2, void* out) {
  dim3 grid((g.N + 31) / 32, (g.M + 31) / 32);
  TB_CUDA(c, launch_k(c, gemm_plain_kernel<EPI, B_MN>, dim3(grid), dim3(256), 0, 1, (const __half*)A, (const __half*)B, (const __half*)B2, out,
                                                            g.M, g.N, g.K));
  TB_CUDA(c, cudaGetLastError());
  return 0;
}

// The instantiated tiles. gate_up: BN <= 128 (its MMA is 2 BN wide); matmul: BN >= 64.
template <int MT, int BN>
int dispatch_epi(Ctx* c, Op& op, Kind kind, const GemmShape& g, int splits, const void* A, const void* B, const void* B2,
                 void* out, bool attr_only) {
  const int epi = epi_of(kind);
  if constexpr (BN == 112) {
    if (epi == EPI_GATE_UP) return run<MT, BN, EPI_GATE_UP, false>(c, op, g, splits, A, B, B2, out, attr_only);
  } else if (kind == K_MATMUL) {
    if constexpr (BN >= 64 && BN != 192) return run<MT, BN, EPI_F16, true>(c, op, g, splits, A, B, B2, out, attr_only);
  } else if (epi == EPI_GATE_UP) {
    if constexpr (BN <= 128) return run<MT, BN, EPI_GATE_UP, false>(c, op, g, splits, A, B, B2, out, attr_only);
  } else if (epi == EPI_ROPE) {
    if constexpr (BN == 128 || BN == 256) return run<MT, BN, EPI_ROPE, false>(c, op, g, splits, A, B, B2, out, attr_only);
  } else if (epi == EPI_F16) {
    return run<MT, BN, EPI_F16, false>(c, op, g, splits, A, B, B2, out, attr_only);
  } else if (epi == EPI_RESID) {
    return run<MT, BN, EPI_RESID, false>(c, op, g, splits, A, B, B2, out, attr_only);
  } else {
    return run<MT, BN, EPI_F32, false>(c, op, g, splits, A, B, B2, out, attr_only);
  }
  return fail(c, "gemm: tile not instantiated for this kernel");
}

int dispatch(Ctx* c, Op& op, Kind kind, int mt, int bn, const GemmShape& g, int splits, const void* A, const void* B,
             const void* B2, void* out, bool attr_only) {
  if (mt == PAIR) {
    if (kind == K_MATMUL) return fail(c, "gemm: CTA pairs take K-major weights only");
    if (bn == 64) return dispatch_pair<64>(c, op, kind, g, splits, A, B, B2, out, attr_only);
    if (bn == 96) return dispatch_pair<96>(c, op, kind, g, splits, A, B, B2, out, attr_only);
    if (bn == 128) return dispatch_pair<128>(c, op, kind, g, splits, A, B, B2, out, attr_only);
    if (bn == 192) return dispatch_pair<192>(c, op, kind, g, splits, A, B, B2, out, attr_only);
    if (bn == 224) return dispatch_pair<224>(c, op, kind, g, splits, A, B, B2, out, attr_only);
    if (bn == 256) return dispatch_pair<256>(c, op, kind, g, splits, A, B, B2, out, attr_only);
    return fail(c, "gemm: no such pair tile");
  }
#define TB_CASE(MT_, BN_) \
  if (mt == MT_ && bn == BN_) return dispatch_epi<MT_, BN_>(c, op, kind, g, splits, A, B, B2, out, attr_only);
  TB_CASE(1, 32) TB_CASE(1, 64) TB_CASE(1, 128) TB_CASE(1, 256)
  TB_CASE(2, 32) TB_CASE(2, 64) TB_CASE(2, 112) TB_CASE(2, 128) TB_CASE(2, 192) TB_CASE(2, 256)
#undef TB_CASE
  return fail(c, "gemm: no such tile");
}

// mt: 1 or 2 = 128-row accumulators of one CTA; PAIR = a CTA pair on a 256-row tile.
struct Plan {
  int mt, bn, splits;
  double t;
};

// Why (MT, BN, splits) cannot run `kind` on this shape, or null when it can: the tile must be
// instantiated for the kernel, its accumulators must fit tensor memory, and a split-K cluster's
// partial tiles must fit the ring they are received in.
const char* plan_error(Kind kind, const GemmShape& g, int mt, int bn, int s) {
  const int epi = epi_of(kind);
  const int bke = g.q8 ? 2 * BK : BK;
  const int nk = (g.K + bke - 1) / bke;
  if (g.q8 && (mt != PAIR || (bn != 128 && bn != 256))) return "FP8 projections run on CTA pairs of 128 or 256 columns";
  // Units of the tile that one CTA must own together, and how many such groups a tile has.
  const int uh = epi == EPI_ROPE ? g.D / 32 : 1;
  if (epi == EPI_ROPE) {
    if (bn != 128 && bn != 256) return "linear_rope_kv tiles are 128 or 256 columns wide";
    if (g.D <= 0 || bn % g.D) return "a linear_rope_kv tile holds whole heads";
  }
  auto recv_fits = [&](int units, int stages, int stage) {
    const int per = ((units / uh + s - 1) / s) * uh;
    // linear_scatter keeps the end of the ring for turning blocks round before they are stored.
    return (s - 1) * per * UNIT_BYTES <= stages * stage - (kind == K_LINEAR_SCATTER ? SCATTER_STAGE_BYTES : 0);
  };
  if (mt == PAIR) {
    if (kind == K_MATMUL) return "CTA pairs take K-major weights only";
    if (bn != 64 && bn != 96 && bn != 128 && bn != 192 && bn != 224 && bn != 256)
      return "pair tiles are 64, 96, 128, 192, 224 or 256 columns wide";
    const int nops = epi == EPI_GATE_UP ? 2 : 1;
    const int stage = BM * BK * 2 + nops * (bn / 2) * BK * 2;
    int stages = (196 * 1024) / stage;
    if (stages > 8) stages = 8;
    if (s < 1 || s > 4) return "splits is 1 to 4 with CTA pairs (a cluster of at most 8)";
    if (s > 1) {
      const int units = bn / 32;
      if (epi == EPI_GATE_UP) return "gate_up does not split K";
      if (s > nk) return "more splits than 64-wide K blocks";
      if ((units / uh) % s) return "splits must divide the tile's 128 x 32 units (its heads, for linear_rope_kv)";
      if (!recv_fits(units, stages, stage)) return "the partial tiles of the other splits do not fit the ring";
    }
    return nullptr;
  }
  if (mt != 1 && mt != 2) return "MT is 1, 2 or 3 (3 = a CTA pair on a 256-row tile)";
  if (bn != 32 && bn != 64 && bn != 112 && bn != 128 && bn != 192 && bn != 256) return "BN is 32, 64, 112, 128, 192 or 256";
  if (bn == 112 && (epi != EPI_GATE_UP || mt != 2)) return "the 112-column tile exists for gate_up with MT = 2 only";
  if (bn == 192 && mt != 2) return "the 192-column tile exists with MT = 2 only";
  if (kind == K_MATMUL && (bn < 64 || bn == 192)) return "matmul tiles are 64, 128 or 256 columns wide";
  if (epi == EPI_GATE_UP && bn > 128) return "gate_up tiles are at most 128 columns wide (its MMA is 2 BN wide)";
  const int nb = bn * (epi == EPI_GATE_UP ? 2 : 1);
  if (mt * nb > 512) return "the accumulators exceed the 512 columns of tensor memory";
  const int stage = mt * BM * BK * 2 + nb * BK * 2;
  int stages = (196 * 1024) / stage;
  if (stages > 8) stages = 8;
  if (stages < 2) return "fewer than two ring stages fit shared memory";
  if (s < 1 || s > 8) return "splits is 1 to 8 (the portable cluster size)";
  if (s > 1) {
    const int units = mt * (bn / 32);
    if (epi == EPI_GATE_UP) return "gate_up does not split K";
    if (s > nk) return "more splits than 64-wide K blocks";
    if ((units / uh) % s) return "splits must divide the tile's 128 x 32 units (its heads, for linear_rope_kv)";
    if (!recv_fits(units, stages, stage)) return "the partial tiles of the other splits do not fit the ring";
  }
  return nullptr;
}

// Picks (MT, BN, splits) by a small cost model: waves of CTAs over the SMs, each CTA bound by
// the slower of its L2-to-SM feed and its MMAs, plus its epilogue (and the partial exchange).
// Returns the candidates, cheapest first.
std::vector<Plan> plan_gemm(Kind kind, const GemmShape& g, int sms) {
  const double FEED = 90e9, TENSOR = 1636e12 / 148.0, HBM = 6.5e12;
  const int nk = (g.K + (g.q8 ? 2 * BK : BK) - 1) / (g.q8 ? 2 * BK : BK);
  const int epi = epi_of(kind);
  const int out_bytes = epi == EPI_RESID ? 8 : (epi == EPI_F32 ? 4 : 2);
  const int nbf = epi == EPI_GATE_UP ? 2 : 1;
  // The 112-column gate_up tile is instantiated but measured slower than 128 at the decode
  // shapes (128 CTAs of 224 MMA columns against 112 CTAs of 256), so only a forced plan picks it.
  const int bns[] = {256, 192, 128, 64, 32};
  std::vector<Plan> all;
  for (int mt = 1; mt <= 2; ++mt) {
    if (mt == 2 && g.M <= BM) continue;
    for (int bn : bns) {
      for (int s = 1; s <= 4; s *= 2) {
        if (plan_error(kind, g, mt, bn, s)) continue;  // (leaves linear_rope_kv its 128- and 256-column tiles)
        if (s > 1 && nk < 8 * s) continue;
        const int nb = bn * nbf;
        const int stage = mt * BM * BK * 2 + nb * BK * 2;
        const long long mtiles = (g.M + mt * BM - 1) / (mt * BM), ntiles = (g.N + bn - 1) / bn;
        const long long ctas = mtiles * ntiles * s;
        const long long waves = (ctas + sms - 1) / sms;
        const double kiter = (double)((nk + s - 1) / s);
        const double t_feed = kiter * stage / FEED;
        const double t_mma = kiter * (2.0 * mt * BM * nb * BK) / TENSOR;
        double t_epi = (double)mt * BM * bn * out_bytes / FEED;
        if (s > 1) t_epi += 2.0e-6 + 2.0 * (s - 1) / s * mt * BM * bn * 4 / FEED;
        double t = waves * ((t_feed > t_mma ? t_feed : t_mma) + 1.5e-6 + t_epi);
        const double floor_t = (2.0 * g.M * g.K + 2.0 * nbf * (double)g.N * g.K + (double)out_bytes * g.M * g.N) / HBM;
        if (t < floor_t) t = floor_t;
        all.push_back({mt, bn, s, t});
      }
    }
  }
  // CTA pairs, for one tile of 129 to 256 rows (a decode step), where they were measured: a CTA
  // takes in 128 rows of activations and half of each weight slice per K step. Clusters of
  // eight (a pair times four splits) measured 40-50 % slower than two splits at every decode
  // shape, so they are left to a forced plan.
  if ((g.q8 || (g.M > BM && g.M <= 2 * BM)) && kind != K_MATMUL) {
    // A streaming kernel draws about 44 GB/s per SM (148 of them make the HBM peak), so a plan
    // is also bounded by the SMs it occupies: hence the tiles between the powers of two (64
    // pairs of 224 gate_up columns against 56 of 256; 64 pairs of 96 QKV columns).
    const double SM_FEED = 44e9;
    for (int bn : {256, 224, 192, 128, 96, 64}) {
      for (int s = 1; s <= 2; s *= 2) {
        if (plan_error(kind, g, PAIR, bn, s)) continue;
        if (s > 1 && nk < 8 * s) continue;
        const int stage = BM * BK * 2 + nbf * (bn / 2) * BK * 2;
        const long long ctas = 2LL * ((g.M + 2 * BM - 1) / (2 * BM)) * ((g.N + bn - 1) / bn) * s;
        const long long waves = (ctas + sms - 1) / sms;
        if (waves > 1 && bn < 128) continue;  // narrow tiles only where they fill one wave
        const double kiter = (double)((nk + s - 1) / s);
        const double t_feed = kiter * stage / FEED;
        const double t_mma = kiter * (2.0 * BM * nbf * bn * BK) / TENSOR;
        double t_epi = (double)BM * bn * out_bytes / FEED;
        if (s > 1) t_epi += 2.0e-6 + 2.0 * (s - 1) / s * BM * bn * 4 / FEED;
        double t = waves * ((t_feed > t_mma ? t_feed : t_mma) + 2.0e-6 + t_epi);
        const double dram = 2.0 * g.M * g.K + 2.0 * nbf * (double)g.N * g.K + (double)out_bytes * g.M * g.N;
        const double floor_t = dram / ((ctas < sms ? ctas : sms) * SM_FEED);
        if (t < floor_t) t = floor_t;
        all.push_back({PAIR, bn, s, t});
      }
    }
  }
  std::stable_sort(all.begin(), all.end(), [](const Plan& a, const Plan& b) { return a.t < b.t; });
  if (all.empty()) all.push_back({1, 64, 1, 1e30});
  return all;
}

}  // namespace

// op.p0: 1 = tcgen05 path, 0 = plain path, -1 = nothing to do. op.p1 = MT, p2 = BN, p3 = splits.
int make_gemm(Ctx* c, Op& op) {
  const auto& s = op.shapes;
  auto bad = [&](const char* why) { return fail(c, op.name + ": " + why); };
  if (op.kind == K_LINEAR_ROPE_KV) {
    // X[T,K], W[Wd,K], pos[T], slot[T], C, S [NPOS,D/2], QKV[T,Wd], Q[T,H,D], Kc, Vc [NS,G,D], K, V [T,G,D]
    if (s[0].size() != 2 || s[1].size() != 2 || s[4].size() != 2 || s[6].size() != 2 || s[7].size() != 3 ||
        s[8].size() != 3 || s[10].size() != 3)
      return bad("shapes are X[T,K], W[Wd,K], pos[T], slot[T], C, S[NPOS,D/2], QKV[T,Wd], Q[T,H,D], Kc, Vc[NS,G,D], K, V[T,G,D]");
    const int64_t T = s[0][0], Wd = s[1][0], H = s[7][1], D = s[7][2], G = s[8][1];
    if (s[1][1] != s[0][1] || s[2][0] != T || s[3][0] != T || s[6][0] != T || s[6][1] != Wd || s[7][0] != T ||
        s[5] != s[4] || s[9] != s[8] || s[11] != s[10] || s[8][2] != D || s[10][0] != T || s[10][1] != G ||
        s[10][2] != D || s[4][1] != D / 2)
      return bad("shapes disagree");
    if (Wd != (H + 2 * G) * D) return bad("W must have (H + 2G) * D rows");
    if (D != 64 && D != 128) return bad("head_dim must be 64 or 128 (use linear and rope_kv otherwise)");
    if (s[0][1] <= 0 || s[0][1] % 8) return bad("K must be a positive multiple of 8 (use linear and rope_kv otherwise)");
    op.rope.H = (int)H, op.rope.G = (int)G, op.rope.D = (int)D, op.rope.NPOS = (int)s[4][0], op.rope.NS = (int)s[8][0];
  }
  const bool q8kind = op.kind == K_LINEAR_Q8 || op.kind == K_LINEAR_RESIDUAL_Q8 || op.kind == K_GATE_UP_Q8;
  for (size_t i = 0; i < s.size() && op.kind != K_LINEAR_ROPE_KV && !q8kind; ++i)
    if (s[i].size() != 2 && !(op.kind == K_LINEAR_SCATTER && i == 2)) return bad("every array is two-dimensional");
  if (q8kind && (s[0].size() != 2 || s[2].size() != 2)) return bad("Xq and Wq are two-dimensional");
  const GemmShape g = gemm_shape(op);
  if (op.kind == K_LINEAR_ROPE_KV) {
    // checked above
  } else if (g.q8) {
    const bool gu = op.kind == K_GATE_UP_Q8;
    const size_t o = gu ? 6 : 4;
    if (s[1].size() != 1 || s[1][0] != g.M || s[2].size() != 2 || s[2][1] != g.K || s[3].size() != 1 || s[3][0] != g.N ||
        (gu && (s[4] != s[2] || s[5] != s[3])) || s[o].size() != 2 || s[o][0] != g.M || s[o][1] != g.N)
      return bad("shapes are Xq[M,K], sx[M], Wq[N,K], sw[N], (Wuq[N,K], su[N],) Y[M,N]");
    if (g.K <= 0 || g.K % 16 || g.N % 8) return bad("K must be a positive multiple of 16 and N a multiple of 8");
  } else if (op.kind == K_LINEAR_SCATTER) {
    if (s[1][1] != g.K || s[2].size() != 1 || (size_t)s[2][0] < sizeof(TpTable))
      return bad("shapes are X[M,K], W[N,K], table[bytes of tb200_tp_sizes]");
    if (g.K <= 0 || g.K % 8 || g.N % 4) return bad("K must be a positive multiple of 8 and N a multiple of 4");
  } else if (op.kind == K_MATMUL) {
    if (s[1][0] != g.K || s[2][0] != g.M || s[2][1] != g.N) return bad("shapes are A[M,K], B[K,N], C[M,N]");
  } else if (op.kind == K_GATE_UP) {
    if (s[1][1] != g.K || s[2] != s[1] || s[3][0] != g.M || s[3][1] != g.N)
      return bad("shapes are X[M,K], Wg[F,K], Wu[F,K], Y[M,F]");
  } else {
    if (s[1][1] != g.K || s[2][0] != g.M || s[2][1] != g.N) return bad("shapes are X[M,K], W[N,K], Y[M,N]");
  }
  if (g.M == 0 || g.N == 0) {
    op.p0 = -1;
    return 0;
  }
  const bool tma_ok = g.K > 0 && g.K % 8 == 0 && (op.kind != K_MATMUL || g.N % 8 == 0);
  op.p0 = tma_ok ? 1 : 0;
  if (!tma_ok) return 0;
  Plan pl = plan_gemm(op.kind, g, c->sm_count)[0];
  // TB200_GEMM_PLAN="mt,bn,splits" overrides the choice (tuning and tests). A value that does
  // not parse, or a tile this kernel and shape cannot run, is an error: a mistyped plan must not
  // pass a test on the default tile.
  if (const char* e = getenv("TB200_GEMM_PLAN")) {
    int a = 0, b = 0, d = 0;
    char tail = 0;
    if (sscanf(e, "%d,%d,%d%c", &a, &b, &d, &tail) != 3)
      return bad((std::string("TB200_GEMM_PLAN=\"") + e + "\" is not MT,BN,splits").c_str());
    if (const char* why = plan_error(op.kind, g, a, b, d))
      return bad((std::string("TB200_GEMM_PLAN=\"") + e + "\": " + why).c_str());
    pl = {a, b, d, 0.0};
  }
  op.p1 = pl.mt;
  op.p2 = pl.bn;
  op.p3 = pl.splits;
  return dispatch(c, op, op.kind, pl.mt, pl.bn, g, pl.splits, nullptr, nullptr, nullptr, nullptr, true);
}

namespace {

// One launch of `op` with plan (mt, bn, splits) on the launch arguments `a`.
int launch_plan(Ctx* c, Op& op, const uint64_t* a, int mt, int bn, int splits) {
  const GemmShape g = gemm_shape(op);
  if (op.kind == K_LINEAR_SCATTER) {
    op.aux = (int)(uint32_t)a[3];
    if (op.aux < 0 || op.aux > 1) return fail(c, op.name + ": which is 0 or 1");
  }
  if (g.q8) {
    // Xq, sx, Wq, sw, (Wuq, su,) out
    const bool gu = op.kind == K_GATE_UP_Q8;
    op.q8[0] = (const float*)a[1], op.q8[1] = (const float*)a[3], op.q8[2] = gu ? (const float*)a[5] : nullptr;
    return dispatch(c, op, op.kind, mt, bn, g, splits, (const void*)a[0], (const void*)a[2],
                    gu ? (const void*)a[4] : nullptr, (void*)a[gu ? 6 : 4], false);
  }
  if (op.kind == K_LINEAR_ROPE_KV) {
    // X, W, pos, slot, C, S, QKV, Q, Kc, Vc, K, V
    RopeArgs& r = op.rope;
    r.pos = (const int*)a[2], r.slot = (const int*)a[3], r.Ct = (const float*)a[4], r.St = (const float*)a[5];
    r.Q = (__half*)a[7], r.Kc = (__half*)a[8], r.Vc = (__half*)a[9], r.Kd = (__half*)a[10], r.Vd = (__half*)a[11];
    return dispatch(c, op, op.kind, mt, bn, g, splits, (const void*)a[0], (const void*)a[1], nullptr, (void*)a[6], false);
  }
  const void* A = (const void*)a[0];
  const void* B = (const void*)a[1];
  const void* B2 = op.kind == K_GATE_UP ? (const void*)a[2] : nullptr;
  void* out = (void*)a[op.kind == K_GATE_UP ? 3 : 2];
  return dispatch(c, op, op.kind, mt, bn, g, splits, A, B, B2, out, false);
}

}  // namespace

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
    r = launch_plan(c, op, a, op.p1, op.p2, op.p3);
  }
  if (r) return r;
  c->launches += 1;
  return 0;
}

// Engine::mm of the reference (src/llm/engine.rs:233-270): the candidate tiles of a projection
// are timed on the device, on the caller's own buffers, and the fastest is kept for every later
// launch of the op. Here the candidates are the cost model's best few (single-CTA tiles, CTA
// pairs, cluster split-K); each is warmed up and then timed launch by launch with the L2
// overwritten in between, because in a decode step the weights always come from HBM while a
// back-to-back loop would serve the smaller projections from the 126 MB L2.
int tune_gemm(Ctx* c, Op& op, const uint64_t* a, float* best_us) {
  if (best_us) *best_us = 0.f;
  if (op.p0 != 1 || getenv("TB200_GEMM_PLAN")) return 0;  // nothing to choose, or the choice is forced
  if (c->capturing) return fail(c, "tb200_tune during graph capture");
  const GemmShape g = gemm_shape(op);
  if (g.K == 0) return 0;
  std::vector<Plan> cands = plan_gemm(op.kind, g, c->sm_count);
  if (cands.size() > 8) cands.resize(8);
  const size_t flush_bytes = (size_t)192 << 20;
  void* flush = nullptr;
  if (cudaMalloc(&flush, flush_bytes) != cudaSuccess) {
    // No room for the buffer that overwrites the L2: time the candidates without it rather than fail.
    cudaGetLastError();
    flush = nullptr;
  }
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  const int WARM = 2, ITERS = 5;
  float best = 1e30f;
  Plan pick = {op.p1, op.p2, op.p3, 0.0};
  int rc = 0;
  for (const Plan& pl : cands) {
    if (dispatch(c, op, op.kind, pl.mt, pl.bn, g, pl.splits, nullptr, nullptr, nullptr, nullptr, true)) continue;
    float times[ITERS];
    bool ok = true;
    for (int it = 0; it < WARM + ITERS && ok; ++it) {
      ok = flush == nullptr || cudaMemsetAsync(flush, it, flush_bytes, c->stream) == cudaSuccess;
      ok = ok && cudaEventRecord(e0, c->stream) == cudaSuccess;
      ok = ok && launch_plan(c, op, a, pl.mt, pl.bn, pl.splits) == 0;
      ok = ok && cudaEventRecord(e1, c->stream) == cudaSuccess;
      ok = ok && cudaEventSynchronize(e1) == cudaSuccess;
      float ms = 0.f;
      ok = ok && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess;
      if (ok && it >= WARM) times[it - WARM] = ms;
    }
    if (!ok) {
      rc = cuda_fail(c, cudaGetLastError(), "tb200_tune");
      break;
    }
    c->launches += WARM + ITERS;
    std::sort(times, times + ITERS);
    const float med = times[ITERS / 2];
    if (med < best) {
      best = med;
      pick = pl;
    }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaStreamSynchronize(c->stream);
  if (flush) cudaFree(flush);
  if (rc) return rc;
  op.p1 = pick.mt;
  op.p2 = pick.bn;
  op.p3 = pick.splits;
  if (best_us && best < 1e29f) *best_us = best * 1000.f;
  return 0;
}

}  // namespace tb
