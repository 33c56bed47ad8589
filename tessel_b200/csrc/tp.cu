// Tensor-parallel exchange fused with the residual add and the next RMSNorm.
//
// Under tensor parallelism o_proj and down_proj leave, on every rank, an f32 partial product
// part[T, dim] whose sum over ranks must be added to the residual stream x and then normalised
// into h for the next projection. The plain path does that with four launches: linear_f32, an
// NCCL allreduce, residual_add, rmsnorm. `tp_reduce_norm` does the last three in ONE kernel over
// peer memory (buffers of the other ranks mapped through CUDA IPC and reached over NVLink with
// ordinary loads; no multicast, no TMA, and no stores into a peer's memory other than flags):
//
//   1. every CTA tells the same-numbered CTA of every peer that this rank's partial is
//      complete (the kernel runs behind the rank's GEMM on the same stream) and waits for theirs;
//   2. row r of the step belongs to rank r % n: its owner loads that row of all n partials
//      (peers' over NVLink), adds them in rank order to its x row, normalises, and stores the
//      new x row and h row in ITS OWN memory (the reduce-scatter);
//   3. every CTA copies the other owners' h rows from their memory into its own h (the
//      all-gather, pulled: a pushed copy would need a system-wide fence that waits for every
//      remote store to be acknowledged, measured at 6-9 us per call). The owner publishes a row
//      in a staging buffer whose every 8 bytes hold two halves and the call's epoch, written
//      and read as ONE 64-bit value each (a single-copy-atomic access: payload and tag cannot be
//      seen torn), so a reader knows from the data itself whether it is current and polls the
//      row directly: no "rows are ready" flag, no release fence.
//
// Between layers only h is gathered: the residual stream stays distributed (a rank's x is
// current in the rows it owns), because nothing but this kernel reads it. The last call of a
// step (do_norm = 0) gathers x instead, for the final norm and the LM head, behind a second
// flag exchange ("my rows are ready", a release), and closes with a third ("I have finished
// reading"): the peers copy the rows straight out of this rank's x, and the very next kernel of
// a step (embed) overwrites x, so the call may not return before every peer is done with it.
//
// Sums are taken in rank order by one owner, so x and h are bit-identical on all ranks, which
// keeps the ranks' greedy tokens in lockstep. Flag waits are bounded: on time-out the kernel
// raises the context's status word and returns.
//
// Why the partial and staging buffers can be reused without a closing barrier: a rank
// overwrites its partial, or its staged rows, only after step 1 of a later call, i.e. after
// every peer has begun that call and therefore finished reading in this one. (x is the
// exception, hence the third exchange above.)
//
// Step 1's signal is a relaxed store: what it announces was written by the PREVIOUS kernel of
// the stream, and a kernel's global writes are complete and visible system-wide when its
// successor starts (the stream order; with programmatic dependent launch, after
// griddepcontrol.wait). No fence of this kernel could add anything to that.
#include "common.cuh"

namespace tb {

namespace {

constexpr int TP_MAX = 8;
constexpr int TP_SLOTS = 4096;  // CTAs a launch may have (rows of the largest step / ranks)
constexpr int TP_THREADS = 1024;
constexpr int TP_PHASES = 4;  // flag words per (slot, sender): partial ready, x rows ready, done reading, spare

// Lives in device memory; written once by the host after the ranks exchanged IPC handles.
struct TpTable {
  float* part[2][TP_MAX];   // the two partial-product buffers of every rank
  float* x[TP_MAX];         // residual stream of every rank
  __half* h[TP_MAX];        // normalised activations of every rank
  uint4* stage[TP_MAX];     // [T, dim/4]: a rank's own h rows as two 64-bit units {2 halves | epoch << 32}
  unsigned int* flags[TP_MAX];  // [TP_SLOTS][TP_PHASES][TP_MAX senders]
  unsigned int* epoch;      // [TP_SLOTS], local: launches this slot has taken part in
  int rank, nranks;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_relaxed_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Loads that always go to the owner's L2 (never a stale line of this SM's L1).
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
__device__ __forceinline__ Unit2 ld_sys_units(const uint4* p) {
  Unit2 v;
  asm volatile("ld.relaxed.sys.global.v2.b64 {%0,%1}, [%2];" : "=l"(v.a), "=l"(v.b) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_units(uint4* p, unsigned int lo0, unsigned int lo1, unsigned int tag) {
  const unsigned long long a = (unsigned long long)lo0 | ((unsigned long long)tag << 32);
  const unsigned long long b = (unsigned long long)lo1 | ((unsigned long long)tag << 32);
  asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1,%2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}

// Thread `tid` < nranks signals peer `tid` and waits for peer `tid`'s signal of this epoch.
// `release`: the signal publishes stores of this CTA (made before the preceding __syncthreads);
// without it the signal only says that the previous kernel of this stream has completed.
__device__ __forceinline__ void exchange_flags(const TpTable& tb_, int slot, int phase, unsigned int epoch,
                                               bool release, unsigned int* status, unsigned int code) {
  const int tid = threadIdx.x;
  if (tid < tb_.nranks && tid != tb_.rank) {
    unsigned int* theirs = tb_.flags[tid] + ((size_t)slot * TP_PHASES + phase) * TP_MAX + tb_.rank;
    if (release)
      st_release_sys(theirs, epoch);
    else
      st_relaxed_sys(theirs, epoch);
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

template <int PER>  // float4 chunks per thread: dim <= PER * 4096
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
  TP_TRACE(0);
  // 1. The partials were written by the previous kernel of each rank's stream, which has
  // completed (and flushed to that rank's L2, where peers read them) before this one signals.
  exchange_flags(tb_, blockIdx.x, 0, epoch, false, status, 401);
  __syncthreads();
  TP_TRACE(1);

  // 2. This rank's rows.
  for (int row = blockIdx.x * n + rank; row < T; row += gridDim.x * n) {
    float4 acc[PER];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = (threadIdx.x + i * TP_THREADS) * 4;
      if (c < dim) {
        const size_t o = (size_t)row * dim + c;
        float4 part[TP_MAX];
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r)
          if (r < n) part[r] = ld_sys_f4(tb_.part[which][r] + o);
        float4 s = part[0];
#pragma unroll
        for (int r = 1; r < TP_MAX; ++r)
          if (r < n) {
            s.x = __fadd_rn(s.x, part[r].x);
            s.y = __fadd_rn(s.y, part[r].y);
            s.z = __fadd_rn(s.z, part[r].z);
            s.w = __fadd_rn(s.w, part[r].w);
          }
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
      }
    }
    if (do_norm) {
      // Block sum of squares (kernels/llm.tl:23), then x * rsqrt(ms + eps) * w.
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = red[threadIdx.x & 31];
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
          st_sys_units(tb_.stage[rank] + (((size_t)row * dim + c) >> 2), y.x, y.y, epoch);
        }
      }
    }
  }
  TP_TRACE(2);
  if (do_norm) {
    // 3a. The other owners' h rows, polled until both halves of a 16-byte unit carry this epoch.
    for (int base = blockIdx.x * n; base < T; base += gridDim.x * n) {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int c = (threadIdx.x + i * TP_THREADS) * 4;
        if (c < dim) {
          Unit2 v[TP_MAX];
          unsigned int pending = 0;
          auto current = [&](const Unit2& u) {
            return (unsigned int)(u.a >> 32) == epoch && (unsigned int)(u.b >> 32) == epoch;
          };
#pragma unroll
          for (int r = 0; r < TP_MAX; ++r)
            if (r < n && r != rank && base + r < T) {
              v[r] = ld_sys_units(tb_.stage[r] + (((size_t)(base + r) * dim + c) >> 2));
              if (!current(v[r])) pending |= 1u << r;
            }
          if (pending) {
            const unsigned long long t0 = globaltimer();
            unsigned int spins = 0;
            while (pending) {
#pragma unroll
              for (int r = 0; r < TP_MAX; ++r)
                if (pending & (1u << r)) {
                  v[r] = ld_sys_units(tb_.stage[r] + (((size_t)(base + r) * dim + c) >> 2));
                  if (current(v[r])) pending &= ~(1u << r);
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
#pragma unroll
          for (int r = 0; r < TP_MAX; ++r)
            if (r < n && r != rank && base + r < T)
              *reinterpret_cast<uint2*>(tb_.h[rank] + (size_t)(base + r) * dim + c) =
                  make_uint2((unsigned int)v[r].a, (unsigned int)v[r].b);
        }
      }
    }
    TP_TRACE(3);
  } else {
    // 3b. Publish this CTA's x rows (the release orders the CTA's stores, made before the
    // barrier, ahead of the flag), wait for the other owners, and copy their rows.
    __syncthreads();
    exchange_flags(tb_, blockIdx.x, 1, epoch, true, status, 403);
    __syncthreads();
    TP_TRACE(3);
    for (int base = blockIdx.x * n; base < T; base += gridDim.x * n) {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int c = (threadIdx.x + i * TP_THREADS) * 4;
        if (c < dim) {
          float4 v[TP_MAX];
#pragma unroll
          for (int r = 0; r < TP_MAX; ++r)
            if (r < n && r != rank && base + r < T) v[r] = ld_sys_f4(tb_.x[r] + (size_t)(base + r) * dim + c);
#pragma unroll
          for (int r = 0; r < TP_MAX; ++r)
            if (r < n && r != rank && base + r < T)
              *reinterpret_cast<float4*>(tb_.x[rank] + (size_t)(base + r) * dim + c) = v[r];
        }
      }
    }
    // 3c. The peers read this rank's rows out of x itself, which the next step's first kernel
    // overwrites: stay until each of them says it has finished (its loads have returned: the
    // values were stored before its barrier).
    __syncthreads();
    exchange_flags(tb_, blockIdx.x, 2, epoch, false, status, 404);
    __syncthreads();
  }
  TP_TRACE(4);
  if (threadIdx.x == 0) tb_.epoch[blockIdx.x] = epoch;
}

}  // namespace

// Shapes: table u8[bytes], W f16[dim], X f32[T, dim]. Arguments: table, W, X (this rank's own
// residual stream; it must be the buffer the table names), eps, which (0/1: the partial buffer
// this projection wrote), do_norm, nranks (the table's).
int make_tp(Ctx* c, Op& op) {
  const auto& s = op.shapes;
  if (s[0].size() != 1 || s[1].size() != 1 || s[2].size() != 2 || s[1][0] != s[2][1])
    return fail(c, op.name + ": shapes are table[bytes], W[dim], X[T, dim]");
  if ((size_t)s[0][0] < sizeof(TpTable)) return fail(c, op.name + ": the table is too small");
  const int64_t dim = s[2][1];
  if (dim % 4 || dim > 2 * 4 * TP_THREADS) return fail(c, op.name + ": dim must be a multiple of 4, at most 8192");
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
  if (dim <= 4 * TP_THREADS)
    TB_CUDA(c, launch_k(c, tp_reduce_norm_kernel<1>, dim3(grid), dim3(TP_THREADS), 0, 1, (const TpTable*)a[0], (const __half*)a[1], eps, T,
                                                                 dim, which, do_norm, c->status));
  else
    TB_CUDA(c, launch_k(c, tp_reduce_norm_kernel<2>, dim3(grid), dim3(TP_THREADS), 0, 1, (const TpTable*)a[0], (const __half*)a[1], eps, T,
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
    t.stage[r] = (uint4*)stage[r];
    t.flags[r] = (unsigned int*)flags[r];
  }
  t.epoch = (unsigned int*)epoch;
  t.rank = rank;
  t.nranks = nranks;
  memcpy(out, &t, sizeof t);
  return 0;
}

}  // namespace tb
