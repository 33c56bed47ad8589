// Tensor-parallel exchange fused with the residual add and the next RMSNorm.
//
// Under tensor parallelism o_proj and down_proj leave, on every rank, an f32 partial product
// part[T, dim] whose sum over ranks must be added to the residual stream x and then normalised
// into h for the next projection. The plain path does that with four launches: linear_f32, an
// NCCL allreduce, residual_add, rmsnorm. Here the data only ever travels one way over NVLink, in
// stores (buffers of the other ranks are mapped through CUDA IPC; no multicast, no TMA on peer
// memory), and every wait polls LOCAL memory:
//
//   0. (in the projection itself, `linear_scatter`, csrc/gemm.cu) row r of the step belongs to
//      rank r % n: every rank's projection stores its partial of that row straight into the
//      owner's inbox, [source rank][r / n][dim] f32 - the reduce-scatter, overlapped with the
//      projection's own tail;
//   1. `tp_reduce_norm`: every CTA tells the same-numbered CTA of every peer that this rank's
//      projection is complete (the kernel runs behind it on the same stream) and waits for theirs;
//   2. the owner adds the n partials of its rows in rank order (its inbox is local memory) to its
//      x rows, normalises, keeps the new x and h rows, and stores each h row into every peer's
//      landing area as 8-byte units {two halves | the call's epoch << 32}: one 64-bit store
//      each, single-copy atomic, so a unit is either old or complete;
//   3. every CTA polls its own landing area for the other owners' rows until every unit carries
//      this call's epoch, and copies the payloads into h (the all-gather). The data says itself
//      when it has arrived: no "rows are ready" flag, no fence over outstanding remote stores
//      (a pushed copy closed by a barrier was measured: its system-wide fence alone took 6-9 us).
//
// Between layers only h is gathered: the residual stream stays distributed (a rank's x is
// current in the rows it owns), because nothing but this kernel reads it. The last call of a
// step (do_norm = 0) gathers x instead, for the final norm and the LM head, the same way with one
// f32 per unit.
//
// Sums are taken in rank order by one owner, so x and h are bit-identical on all ranks, which
// keeps the ranks' greedy tokens in lockstep. Waits are bounded: on time-out the kernel raises
// the context's status word and returns.
//
// Why nothing needs a closing barrier: a rank stores into a peer's inbox or landing area only
// after step 1 of a later call (the projection that fills inbox w runs behind the call that
// used inbox 1 - w), i.e. after that peer has begun the later call and therefore finished
// reading in this one. Nobody reads another rank's x, h or inbox.
//
// Step 1's signal is a relaxed store: what it announces was written by the PREVIOUS kernel of
// the stream, and a kernel's writes, those into a peer's memory included, are complete when its
// successor starts (the stream order; with programmatic dependent launch, after
// griddepcontrol.wait, which returns only once the earlier grid has finished and its memory
// operations are performed).
#include "common.cuh"

namespace tb {

namespace {

constexpr int TP_SLOTS = 4096;  // CTAs a launch may have (rows of the largest step / ranks)
constexpr int TP_THREADS = 512;  // 128 registers a thread: the gather keeps eight owners' units in flight
constexpr int TP_PHASES = 4;  // flag words per (slot, sender): projection complete; three spare

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Loads that always go to L2, where stores from other GPUs land (never a stale line of this SM's L1).
__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Two 64-bit units {payload | tag << 32}: each unit is one scalar access, so its payload and its
// tag are always from the same store.
struct Unit2 {
  unsigned long long a, b;
};
__device__ __forceinline__ Unit2 ld_sys_units(const unsigned long long* p) {
  Unit2 v;
  asm volatile("ld.relaxed.sys.global.v2.b64 {%0,%1}, [%2];" : "=l"(v.a), "=l"(v.b) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_units(unsigned long long* p, unsigned int lo0, unsigned int lo1,
                                             unsigned int tag) {
  const unsigned long long a = (unsigned long long)lo0 | ((unsigned long long)tag << 32);
  const unsigned long long b = (unsigned long long)lo1 | ((unsigned long long)tag << 32);
  asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1,%2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}

// Thread `tid` < nranks signals peer `tid` and waits for peer `tid`'s signal of this epoch.
__device__ __forceinline__ void exchange_flags(const TpTable& tb_, int slot, int phase, unsigned int epoch,
                                               unsigned int* status, unsigned int code) {
  const int tid = threadIdx.x;
  if (tid < tb_.nranks && tid != tb_.rank) {
    st_relaxed_sys(tb_.flags[tid] + ((size_t)slot * TP_PHASES + phase) * TP_MAX + tb_.rank, epoch);
    const unsigned int* mine = tb_.flags[tb_.rank] + ((size_t)slot * TP_PHASES + phase) * TP_MAX + tid;
    const unsigned long long t0 = globaltimer();
    unsigned int spins = 0;
    // Epochs only grow; a peer that is a launch ahead has already passed this one.
    while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 255u) == 0) {
        if (*(volatile unsigned int*)status != 0) break;
        if (globaltimer() - t0 > WAIT_LIMIT_NS / 2) {
          atomicCAS(status, 0u, code);
          break;
        }
      }
    }
  }
}

#ifdef TB200_TRACE
// Development builds: %globaltimer stamps of CTA 0's thread 0 in the unused tail of this rank's flag buffer.
#define TP_TRACE(k)                                                                                      \
  do {                                                                                                   \
    if (blockIdx.x == 0 && threadIdx.x == 0)                                                             \
      reinterpret_cast<unsigned long long*>(tb_.flags[tb_.rank] + (size_t)(TP_SLOTS - 64) * TP_PHASES * TP_MAX)[k] = globaltimer(); \
  } while (0)
#else
#define TP_TRACE(k) \
  do {              \
  } while (0)
#endif

__device__ __forceinline__ bool current(const Unit2& u, unsigned int epoch) {
  return (unsigned int)(u.a >> 32) == epoch && (unsigned int)(u.b >> 32) == epoch;
}

// Reads, for every other owner r, the two units at `land + (base + r) * row_units + off` of this
// rank's landing area, polling until they carry `epoch` (all loads are issued before any is
// tested: the rows mostly arrive together). Returns the owners whose units never came.
__device__ __forceinline__ unsigned int gather_units(const unsigned long long* land, size_t row_units, size_t off,
                                                     int base, int T, int n, int rank, unsigned int epoch,
                                                     Unit2 (&v)[TP_MAX], unsigned int* status) {
  unsigned int pending = 0;
#pragma unroll
  for (int r = 0; r < TP_MAX; ++r)
    if (r < n && r != rank && base + r < T) {
      v[r] = ld_sys_units(land + (size_t)(base + r) * row_units + off);
      if (!current(v[r], epoch)) pending |= 1u << r;
    }
  if (pending) {
    const unsigned long long t0 = globaltimer();
    unsigned int spins = 0;
    while (pending) {
#pragma unroll
      for (int r = 0; r < TP_MAX; ++r)
        if (pending & (1u << r)) {
          v[r] = ld_sys_units(land + (size_t)(base + r) * row_units + off);
          if (current(v[r], epoch)) pending &= ~(1u << r);
        }
      if ((++spins & 63u) == 0) {
        if (*(volatile unsigned int*)status != 0) break;
        if (globaltimer() - t0 > WAIT_LIMIT_NS / 2) {
          atomicCAS(status, 0u, 402u);
          break;
        }
      }
    }
  }
  return pending;
}

template <int PER>  // float4 chunks per thread: dim <= PER * 4 * TP_THREADS
__global__ void __launch_bounds__(TP_THREADS, 1)
    tp_reduce_norm_kernel(const TpTable* __restrict__ table, const __half* __restrict__ W, float eps, int T, int dim,
                          int which, int do_norm, unsigned int* status) {
  pdl_launch();
  pdl_wait();
  __shared__ TpTable tb_;
  __shared__ float red[32];
  __shared__ unsigned int s_epoch;
  static_assert(sizeof(TpTable) % 8 == 0, "the table is copied in 8-byte words");
  if (threadIdx.x < sizeof(TpTable) / 8)
    reinterpret_cast<unsigned long long*>(&tb_)[threadIdx.x] =
        reinterpret_cast<const unsigned long long*>(table)[threadIdx.x];
  __syncthreads();
  if (threadIdx.x == 0) s_epoch = tb_.epoch[blockIdx.x] + 1;
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const int n = tb_.nranks, rank = tb_.rank;
  const int per = (T + n - 1) / n;  // rows of a source's share of an inbox
  TP_TRACE(0);
  // 1. Every rank's projection (and with it its stores into the owners' inboxes) is complete.
  exchange_flags(tb_, blockIdx.x, 0, epoch, status, 401);
  __syncthreads();
  TP_TRACE(1);

  // 2. This rank's rows: sum the inbox in rank order, add to x, normalise, send to every peer.
  const float* inbox = tb_.part[which][rank];
  for (int row = blockIdx.x * n + rank; row < T; row += gridDim.x * n) {
    const int slot = row / n;
    float4 acc[PER];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = (threadIdx.x + i * TP_THREADS) * 4;
      if (c < dim) {
        float4 part[TP_MAX];
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r)
          if (r < n) part[r] = ld_sys_f4(inbox + ((size_t)r * per + slot) * dim + c);
        float4 s = part[0];
#pragma unroll
        for (int r = 1; r < TP_MAX; ++r)
          if (r < n) {
            s.x = __fadd_rn(s.x, part[r].x);
            s.y = __fadd_rn(s.y, part[r].y);
            s.z = __fadd_rn(s.z, part[r].z);
            s.w = __fadd_rn(s.w, part[r].w);
          }
        const size_t o = (size_t)row * dim + c;
        float4 x = *reinterpret_cast<const float4*>(tb_.x[rank] + o);
        x.x = __fadd_rn(x.x, s.x);
        x.y = __fadd_rn(x.y, s.y);
        x.z = __fadd_rn(x.z, s.z);
        x.w = __fadd_rn(x.w, s.w);
        acc[i] = x;
        *reinterpret_cast<float4*>(tb_.x[rank] + o) = x;
        ss += __fmul_rn(x.x, x.x);
        ss += __fmul_rn(x.y, x.y);
        ss += __fmul_rn(x.z, x.z);
        ss += __fmul_rn(x.w, x.w);
        if (!do_norm) {
          // The last call of a step: every rank gets the finished x row, one f32 per unit.
#pragma unroll
          for (int r = 0; r < TP_MAX; ++r)
            if (r < n && r != rank) {
              unsigned long long* dst = tb_.stage[r] + o;
              st_sys_units(dst, __float_as_uint(x.x), __float_as_uint(x.y), epoch);
              st_sys_units(dst + 2, __float_as_uint(x.z), __float_as_uint(x.w), epoch);
            }
        }
      }
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
          *reinterpret_cast<uint2*>(tb_.h[rank] + (size_t)row * dim + c) = y;
          // Units c/2 and c/2 + 1 of the row in every peer's landing area.
#pragma unroll
          for (int r = 0; r < TP_MAX; ++r)
            if (r < n && r != rank) st_sys_units(tb_.stage[r] + (size_t)row * dim + (c >> 1), y.x, y.y, epoch);
        }
      }
    }
  }
  TP_TRACE(2);
  // 3. The other owners' rows, from this rank's own landing area.
  const unsigned long long* land = tb_.stage[rank];
  for (int base = blockIdx.x * n; base < T; base += gridDim.x * n) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = (threadIdx.x + i * TP_THREADS) * 4;
      if (c >= dim) continue;
      Unit2 v[TP_MAX];
      if (do_norm) {
        gather_units(land, (size_t)dim, (size_t)(c >> 1), base, T, n, rank, epoch, v, status);
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r)
          if (r < n && r != rank && base + r < T)
            *reinterpret_cast<uint2*>(tb_.h[rank] + (size_t)(base + r) * dim + c) =
                make_uint2((unsigned int)v[r].a, (unsigned int)v[r].b);
      } else {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          gather_units(land, (size_t)dim, (size_t)(c + 2 * half), base, T, n, rank, epoch, v, status);
#pragma unroll
          for (int r = 0; r < TP_MAX; ++r)
            if (r < n && r != rank && base + r < T)
              *reinterpret_cast<float2*>(tb_.x[rank] + (size_t)(base + r) * dim + c + 2 * half) =
                  make_float2(__uint_as_float((unsigned int)v[r].a), __uint_as_float((unsigned int)v[r].b));
        }
      }
    }
  }
  TP_TRACE(3);
  if (threadIdx.x == 0) tb_.epoch[blockIdx.x] = epoch;
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
  // One CTA per row this rank owns; every rank launches the same grid.
  // At most one CTA per SM, so that the CTAs that wait on each other across ranks are all resident.
  int grid = (T + nranks - 1) / nranks;
  if (grid > c->sm_count) grid = c->sm_count;
  if (grid > TP_SLOTS) grid = TP_SLOTS;
  if (dim <= 2 * 4 * TP_THREADS)
    TB_CUDA(c, launch_k(c, tp_reduce_norm_kernel<2>, dim3(grid), dim3(TP_THREADS), 0, 1, (const TpTable*)a[0], (const __half*)a[1], eps, T,
                                                                 dim, which, do_norm, c->status));
  else
    TB_CUDA(c, launch_k(c, tp_reduce_norm_kernel<4>, dim3(grid), dim3(TP_THREADS), 0, 1, (const TpTable*)a[0], (const __half*)a[1], eps, T,
                                                                 dim, which, do_norm, c->status));
  TB_CUDA(c, cudaGetLastError());
  c->launches += 1;
  return 0;
}

size_t tp_table_bytes() { return sizeof(TpTable); }
size_t tp_flag_bytes() { return (size_t)TP_SLOTS * TP_PHASES * TP_MAX * sizeof(unsigned int); }
size_t tp_epoch_bytes() { return (size_t)TP_SLOTS * sizeof(unsigned int); }

// Fills a host copy of the table. Pointer arrays are indexed by rank.
int tp_fill_table(void* out, size_t out_bytes, int rank, int nranks, const uint64_t* part0, const uint64_t* part1,
                  const uint64_t* x, const uint64_t* h, const uint64_t* stage, const uint64_t* flags, uint64_t epoch) {
  if (out_bytes < sizeof(TpTable) || nranks < 1 || nranks > TP_MAX || rank < 0 || rank >= nranks) return 1;
  TpTable t;
  memset(&t, 0, sizeof t);
  for (int r = 0; r < nranks; ++r) {
    t.part[0][r] = (float*)part0[r];
    t.part[1][r] = (float*)part1[r];
    t.x[r] = (float*)x[r];
    t.h[r] = (__half*)h[r];
    t.stage[r] = (unsigned long long*)stage[r];
    t.flags[r] = (unsigned int*)flags[r];
  }
  t.epoch = (unsigned int*)epoch;
  t.rank = rank;
  t.nranks = nranks;
  memcpy(out, &t, sizeof t);
  return 0;
}

}  // namespace tb
