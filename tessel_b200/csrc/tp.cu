// Tensor-parallel exchange fused with the residual add and the next RMSNorm.
//
// Under tensor parallelism o_proj and down_proj leave, on every rank, an f32 partial product
// part[T, dim] whose sum over ranks must be added to the residual stream x and then normalised
// into h for the next projection. The plain path does that with four launches: linear_f32, an
// NCCL allreduce, residual_add, rmsnorm. Here the data only ever travels one way over NVLink, in
// stores (buffers of the other ranks are mapped through CUDA IPC; no multicast, no TMA on peer
// memory), every wait polls LOCAL memory, and the data says itself when it has arrived: there
// are no flags, no barrier and no fence over outstanding remote stores.
//
//   0. (in the projection itself, `linear_scatter`, csrc/gemm.cu) row r of the step belongs to
//      rank r % n: every rank's projection stores its partial of that row straight into the
//      owner's inbox, [source rank][r / n][dim] f32 - the reduce-scatter, overlapped with the
//      projection's own tail;
//   1. `tp_reduce_norm`: the owner polls its inbox (local memory) until the n partials of a row
//      are there, adds them in rank order to its x row, normalises, keeps the new x and h rows,
//      and stores each h row into every peer's landing area;
//   2. every CTA polls its own landing area for the other owners' rows and copies them into h
//      (the all-gather).
//
// "There" means: not TP_EMPTY. Inboxes and landing areas hold the 32-bit pattern TP_EMPTY
// (0xffffffff: as f32, or as two f16, a NaN that no arithmetic instruction produces) wherever
// nothing has arrived; a sender that does have that pattern to send sends another NaN instead;
// and the reader puts TP_EMPTY back into every word it has consumed. A 32-bit word is written by
// one store instruction and is single-copy atomic, so a word is either empty or complete, and
// every word is tested on its own: nothing is assumed about the order in which the words of a
// remote store, or of different stores, become visible. (An earlier form announced the
// projections with per-CTA flags and tagged every 32-bit payload with a 32-bit call counter:
// twice the bytes over NVLink and one more NVLink latency per call. A pushed copy closed by a
// barrier was measured too: its system-wide fence alone took 6-9 us.)
//
// Between layers only h is gathered: the residual stream stays distributed (a rank's x is
// current in the rows it owns), because nothing but this kernel reads it. The last call of a
// step (do_norm = 0) gathers x instead, for the final norm and the LM head, the same way with one
// f32 per word.
//
// Sums are taken in rank order by one owner, so x and h are bit-identical on all ranks, which
// keeps the ranks' greedy tokens in lockstep. Waits are bounded: on time-out the kernel raises
// the context's status word and returns.
//
// Why a word is never overwritten before it has been consumed and emptied. Inboxes alternate
// (`which`): the projection of call k + 2 is the next writer of the inbox call k read. A rank
// reaches that projection only after its own call k + 1 has gathered every owner's rows of call
// k + 1, and an owner sends those only after it has summed the partials of call k + 1 from ALL
// ranks, which every rank produces after finishing call k (one stream per rank). So when any
// rank writes into an inbox for call k + 2, every rank has finished call k. The same chain
// covers the landing area: an owner sends rows of call k + 1 only after every rank's projection
// of call k + 1 has delivered its partials, i.e. after every rank has finished call k and
// emptied what it consumed.
#include "common.cuh"

namespace tb {

namespace {

constexpr int TP_THREADS = 512;  // 128 registers a thread: the polls keep eight ranks' words in flight
constexpr unsigned int TP_EMPTY = 0xffffffffu;
constexpr unsigned int TP_NAN_F32 = 0x7fffffffu;  // sent in place of TP_EMPTY: still a NaN
constexpr unsigned int TP_NAN_H2 = 0x7fff7fffu;   // ... as two halves

// Loads that always go to L2, where stores from other GPUs land (never a stale line of this SM's L1).
__device__ __forceinline__ uint4 ld_sys_u4(const unsigned int* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_sys_u2(const unsigned int* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_u4(unsigned int* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_sys_u2(unsigned int* p, uint2 v) {
  asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ bool landed(const uint4& v) {
  return v.x != TP_EMPTY && v.y != TP_EMPTY && v.z != TP_EMPTY && v.w != TP_EMPTY;
}
__device__ __forceinline__ bool landed(const uint2& v) { return v.x != TP_EMPTY && v.y != TP_EMPTY; }
__device__ __forceinline__ unsigned int sendable(unsigned int w, unsigned int nan) { return w == TP_EMPTY ? nan : w; }

__device__ __forceinline__ uint4 ld_sys(const unsigned int* p, uint4*) { return ld_sys_u4(p); }
__device__ __forceinline__ uint2 ld_sys(const unsigned int* p, uint2*) { return ld_sys_u2(p); }

// Reads one vector (V = uint4 or uint2) at `base + at[r]` for every rank r in `mask`, polling
// until none of its words is TP_EMPTY. All loads are issued before any is tested: the words
// mostly arrive together. Returns the ranks whose words never came (the status word then holds
// `code`, or an earlier failure).
template <typename V>
__device__ __forceinline__ unsigned int poll(const unsigned int* base, const size_t (&at)[TP_MAX], unsigned int mask,
                                             V (&v)[TP_MAX], unsigned int* status, unsigned int code) {
  unsigned int pending = 0;
#pragma unroll
  for (int r = 0; r < TP_MAX; ++r)
    if (mask & (1u << r)) {
      v[r] = ld_sys(base + at[r], (V*)nullptr);
      if (!landed(v[r])) pending |= 1u << r;
    }
  if (pending) {
    const unsigned long long t0 = globaltimer();
    unsigned int spins = 0;
    while (pending) {
#pragma unroll
      for (int r = 0; r < TP_MAX; ++r)
        if (pending & (1u << r)) {
          v[r] = ld_sys(base + at[r], (V*)nullptr);
          if (landed(v[r])) pending &= ~(1u << r);
        }
      if ((++spins & 63u) == 0) {
        if (*(volatile unsigned int*)status != 0) break;
        if (globaltimer() - t0 > WAIT_LIMIT_NS / 2) {
          atomicCAS(status, 0u, code);
          break;
        }
      }
    }
  }
  return pending;
}

#ifdef TB200_TRACE
// Trace builds: %globaltimer stamps of thread 0 of the first TP_TRACE_CTAS CTAs at kernel start,
// when the partials of the CTA's first row have landed, when its rows are sent, and when the
// other owners' rows have landed, for the last two calls: after the TP_TRACE_CTAS call counters
// of the table's `trace` buffer, [call parity][CTA][4] u64.
constexpr int TP_TRACE_CTAS = 64;
#define TP_TRACE(k)                                                                                        \
  do {                                                                                                     \
    if (threadIdx.x == 0 && blockIdx.x < TP_TRACE_CTAS && tb_.trace)                                       \
      reinterpret_cast<unsigned long long*>(tb_.trace + TP_TRACE_CTAS)[((call & 1u) * TP_TRACE_CTAS + blockIdx.x) * 4 + (k)] = \
          globaltimer();                                                                                   \
  } while (0)
#else
#define TP_TRACE(k) \
  do {              \
  } while (0)
#endif

template <int PER>  // float4 chunks per thread: dim <= PER * 4 * TP_THREADS
__global__ void __launch_bounds__(TP_THREADS, 1)
    tp_reduce_norm_kernel(const TpTable* __restrict__ table, const __half* __restrict__ W, float eps, int T, int dim,
                          int which, int do_norm, unsigned int* status) {
  pdl_launch();
  pdl_wait();
  __shared__ TpTable tb_;
  __shared__ float red[32];
  static_assert(sizeof(TpTable) % 8 == 0, "the table is copied in 8-byte words");
  if (threadIdx.x < sizeof(TpTable) / 8)
    reinterpret_cast<unsigned long long*>(&tb_)[threadIdx.x] =
        reinterpret_cast<const unsigned long long*>(table)[threadIdx.x];
  __syncthreads();
  const int n = tb_.nranks, rank = tb_.rank;
  const int per = (T + n - 1) / n;  // rows of a source's share of an inbox
  const unsigned int everyone = (1u << n) - 1u;
#ifdef TB200_TRACE
  unsigned int call = 0;
  if (tb_.trace && blockIdx.x < TP_TRACE_CTAS) call = tb_.trace[blockIdx.x] + 1;
#endif
  TP_TRACE(0);

  // 1. This rank's rows: wait for the n partials, sum them in rank order, add to x, normalise, send.
  unsigned int* inbox = reinterpret_cast<unsigned int*>(tb_.part[which][rank]);
  float* xrow0 = tb_.x;
  bool first = true;
  for (int row = blockIdx.x * n + rank; row < T; row += gridDim.x * n) {
    const int slot = row / n;
    float4 acc[PER];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = (threadIdx.x + i * TP_THREADS) * 4;
      if (c < dim) {
        uint4 part[TP_MAX];
        size_t at[TP_MAX];
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r) at[r] = ((size_t)r * per + slot) * dim + c;
        poll(inbox, at, everyone, part, status, 401u);
        const uint4 empty = make_uint4(TP_EMPTY, TP_EMPTY, TP_EMPTY, TP_EMPTY);
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r)
          if (r < n) *reinterpret_cast<uint4*>(inbox + at[r]) = empty;
        float4 s = make_float4(__uint_as_float(part[0].x), __uint_as_float(part[0].y), __uint_as_float(part[0].z),
                               __uint_as_float(part[0].w));
#pragma unroll
        for (int r = 1; r < TP_MAX; ++r)
          if (r < n) {
            s.x = __fadd_rn(s.x, __uint_as_float(part[r].x));
            s.y = __fadd_rn(s.y, __uint_as_float(part[r].y));
            s.z = __fadd_rn(s.z, __uint_as_float(part[r].z));
            s.w = __fadd_rn(s.w, __uint_as_float(part[r].w));
          }
        const size_t o = (size_t)row * dim + c;
        float4 x = *reinterpret_cast<const float4*>(xrow0 + o);
        x.x = __fadd_rn(x.x, s.x);
        x.y = __fadd_rn(x.y, s.y);
        x.z = __fadd_rn(x.z, s.z);
        x.w = __fadd_rn(x.w, s.w);
        acc[i] = x;
        *reinterpret_cast<float4*>(xrow0 + o) = x;
        ss += __fmul_rn(x.x, x.x);
        ss += __fmul_rn(x.y, x.y);
        ss += __fmul_rn(x.z, x.z);
        ss += __fmul_rn(x.w, x.w);
        if (!do_norm) {
          // The last call of a step: every rank gets the finished x row, one f32 per word.
          const uint4 y = make_uint4(sendable(__float_as_uint(x.x), TP_NAN_F32), sendable(__float_as_uint(x.y), TP_NAN_F32),
                                     sendable(__float_as_uint(x.z), TP_NAN_F32), sendable(__float_as_uint(x.w), TP_NAN_F32));
#pragma unroll
          for (int r = 0; r < TP_MAX; ++r)
            if (r < n && r != rank) st_sys_u4(tb_.stage[r] + o, y);
        }
      }
    }
    if (first) {
      TP_TRACE(1);
      first = false;
    }
    if (do_norm) {
      // Block sum of squares (kernels/llm.tl:23), then x * rsqrt(ms + eps) * w.
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = (threadIdx.x & 31) < TP_THREADS / 32 ? red[threadIdx.x & 31] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
      __syncthreads();
      const float ms = __fdiv_rn(tot, (float)dim);
      const float rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int c = (threadIdx.x + i * TP_THREADS) * 4;
        if (c < dim) {
          const __half2 w01 = *reinterpret_cast<const __half2*>(W + c);
          const __half2 w23 = *reinterpret_cast<const __half2*>(W + c + 2);
          uint2 y;
          y.x = pack_h2(__fmul_rn(__fmul_rn(acc[i].x, rs), __low2float(w01)),
                        __fmul_rn(__fmul_rn(acc[i].y, rs), __high2float(w01)));
          y.y = pack_h2(__fmul_rn(__fmul_rn(acc[i].z, rs), __low2float(w23)),
                        __fmul_rn(__fmul_rn(acc[i].w, rs), __high2float(w23)));
          *reinterpret_cast<uint2*>(tb_.h + (size_t)row * dim + c) = y;
          // Words c/2 and c/2 + 1 of the row ([T][dim / 2] words) in every peer's landing area.
          const uint2 z = make_uint2(sendable(y.x, TP_NAN_H2), sendable(y.y, TP_NAN_H2));
#pragma unroll
          for (int r = 0; r < TP_MAX; ++r)
            if (r < n && r != rank) st_sys_u2(tb_.stage[r] + (size_t)row * (dim >> 1) + (c >> 1), z);
        }
      }
    }
  }
  TP_TRACE(2);
  // 2. The other owners' rows, from this rank's own landing area; what is taken is emptied.
  unsigned int* land = tb_.stage[rank];
  for (int base = blockIdx.x * n; base < T; base += gridDim.x * n) {
    unsigned int mask = 0;
#pragma unroll
    for (int r = 0; r < TP_MAX; ++r)
      if (r < n && r != rank && base + r < T) mask |= 1u << r;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = (threadIdx.x + i * TP_THREADS) * 4;
      if (c >= dim) continue;
      size_t at[TP_MAX];
      if (do_norm) {
        uint2 v[TP_MAX];
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r) at[r] = (size_t)(base + r) * (dim >> 1) + (c >> 1);
        poll(land, at, mask, v, status, 402u);
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r)
          if (mask & (1u << r)) {
            *reinterpret_cast<uint2*>(tb_.h + (size_t)(base + r) * dim + c) = v[r];
            *reinterpret_cast<uint2*>(land + at[r]) = make_uint2(TP_EMPTY, TP_EMPTY);
          }
      } else {
        uint4 v[TP_MAX];
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r) at[r] = (size_t)(base + r) * dim + c;
        poll(land, at, mask, v, status, 402u);
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r)
          if (mask & (1u << r)) {
            *reinterpret_cast<uint4*>(xrow0 + (size_t)(base + r) * dim + c) = v[r];
            *reinterpret_cast<uint4*>(land + at[r]) = make_uint4(TP_EMPTY, TP_EMPTY, TP_EMPTY, TP_EMPTY);
          }
      }
    }
  }
  TP_TRACE(3);
#ifdef TB200_TRACE
  if (threadIdx.x == 0 && tb_.trace && blockIdx.x < TP_TRACE_CTAS) tb_.trace[blockIdx.x] = call;
#endif
}

}  // namespace

// Shapes: table u8[bytes], W f16[dim], X f32[T, dim]. Arguments: table, W, X (this rank's own
// residual stream; it must be the buffer the table names), eps, which (0/1: the inbox the
// projection filled), do_norm, nranks (the table's).
int make_tp(Ctx* c, Op& op) {
  const auto& s = op.shapes;
  if (s[0].size() != 1 || s[1].size() != 1 || s[2].size() != 2 || s[1][0] != s[2][1])
    return fail(c, op.name + ": shapes are table[bytes], W[dim], X[T, dim]");
  if ((size_t)s[0][0] < sizeof(TpTable)) return fail(c, op.name + ": the table is too small");
  const int64_t dim = s[2][1];
  if (dim % 4 || dim > 4 * 4 * TP_THREADS) return fail(c, op.name + ": dim must be a multiple of 4, at most 8192");
  return 0;
}

int launch_tp(Ctx* c, Op& op, const uint64_t* a) {
  const auto& s = op.shapes;
  const int T = (int)s[2][0], dim = (int)s[2][1];
  if (T == 0) return 0;
  const float eps = bits_f32(a[3]);
  const int which = (int)(uint32_t)a[4], do_norm = (int)(uint32_t)a[5];
  if (which < 0 || which > 1) return fail(c, op.name + ": which is 0 or 1");
  const int nranks = (int)(uint32_t)a[6];
  if (nranks < 2 || nranks > TP_MAX) return fail(c, op.name + ": nranks (the table's) is 2 to 8");
  // One CTA per row this rank owns, at most one per SM; every rank launches the same grid, and
  // CTA b of a rank takes the rows CTA b of the owners sends.
  int grid = (T + nranks - 1) / nranks;
  if (grid > c->sm_count) grid = c->sm_count;
  const TpTable* table = (const TpTable*)a[0];
  const __half* W = (const __half*)a[1];
  if (dim <= 2 * 4 * TP_THREADS)
    TB_CUDA(c, launch_k(c, tp_reduce_norm_kernel<2>, dim3(grid), dim3(TP_THREADS), 0, 1, table, W, eps, T, dim, which,
                        do_norm, c->status));
  else
    TB_CUDA(c, launch_k(c, tp_reduce_norm_kernel<4>, dim3(grid), dim3(TP_THREADS), 0, 1, table, W, eps, T, dim, which,
                        do_norm, c->status));
  TB_CUDA(c, cudaGetLastError());
  c->launches += 1;
  return 0;
}

size_t tp_table_bytes() { return sizeof(TpTable); }
// Trace builds: 64 call counters (u32), then [2][64][4] u64 stamps.
size_t tp_trace_bytes() { return 64 * 4 + 2 * 64 * 4 * 8; }

// Fills a host copy of the table. Pointer arrays are indexed by rank.
int tp_fill_table(void* out, size_t out_bytes, int rank, int nranks, const uint64_t* inbox0, const uint64_t* inbox1,
                  const uint64_t* landing, uint64_t x, uint64_t h, uint64_t trace) {
  if (out_bytes < sizeof(TpTable) || nranks < 1 || nranks > TP_MAX || rank < 0 || rank >= nranks) return 1;
  TpTable t;
  memset(&t, 0, sizeof t);
  for (int r = 0; r < nranks; ++r) {
    t.part[0][r] = (float*)inbox0[r];
    t.part[1][r] = (float*)inbox1[r];
    t.stage[r] = (unsigned int*)landing[r];
  }
  t.x = (float*)x;
  t.h = (__half*)h;
  t.trace = (unsigned int*)trace;
  t.rank = rank;
  t.nranks = nranks;
  memcpy(out, &t, sizeof t);
  return 0;
}

}  // namespace tb
