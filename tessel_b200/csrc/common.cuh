// Shared declarations of libtessel_b200: the context behind the C ABI, the op
// table, and the sm_100a PTX wrappers (mbarrier, TMA, tcgen05/TMEM) the kernels
// are written with.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

namespace tb {

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

enum Kind : int {
  K_EMBED = 0,
  K_RMSNORM,
  K_LINEAR,
  K_LINEAR_RESIDUAL,
  K_LOGITS,
  K_GATE_UP,
  K_ROPE_Q,
  K_KV_WRITE,
  K_PREFILL_ATTENTION,
  K_DECODE_ATTENTION,
  K_RMSNORM_ROWS,
  K_MATMUL,
  K_FLASH_ATTENTION,
  K_PAGED_ATTENTION,
  // Extensions beyond the reference's kernel list.
  K_LINEAR_F32,     // Y f32 = X W^T (a tensor-parallel rank's partial product)
  K_RESIDUAL_ADD,   // R f32 += P f32
  K_ARGMAX_ROWS,    // first index of each row's maximum
  K_ROPE_KV,        // rope_q and kv_write in one launch
  K_TP_REDUCE_NORM, // cross-rank sum of partial products + residual add + RMSNorm over peer memory
  K_DECODE_ADVANCE, // next decode step's tok/pos/slot/lens from this step's picks, on the device
  K_ARGMAX_PARTIAL, // a rank's (maximum, index) over its slice of a vocabulary split across ranks
  K_ARGMAX_MERGE,   // first maximum over the ranks' parts
  K_CHUNK_ATTENTION,  // causal attention of a prompt chunk's rows against the paged cache
  K_LINEAR_SCATTER,   // a tensor-parallel rank's partial product, each row stored into its owner rank's memory
  K_LINEAR_ROPE_KV,   // the QKV projection with rope_q and kv_write as its epilogue
  // FP8 mode (non-parity): E4M3 operands with one f32 scale per row, f32 accumulation.
  K_QUANT_ROWS,          // X f16 [M,K] -> Q u8 [M,K], S f32 [M]
  K_RMSNORM_Q8,          // RMSNorm followed by quant_rows of its f16 result
  K_LINEAR_Q8,           // Y f16 = (Xq sx) (Wq sw)^T
  K_LINEAR_RESIDUAL_Q8,  // R f32 += (Xq sx) (Wq sw)^T
  K_GATE_UP_Q8,          // Y f16 = silu((Xq sx)(Wgq sg)^T) * ((Xq sx)(Wuq su)^T)
  K_COUNT
};

// Tensor maps already encoded for an op: they depend only on the op (shapes, tile) and the
// operand addresses, so a launch that sees the same addresses again (layer l of every step)
// reuses them instead of calling cuTensorMapEncodeTiled two or three times.
struct MapEntry {
  uint64_t key[4];
  CUtensorMap m[3];
};

// linear_rope_kv: what the projection's epilogue needs beyond the product (kernels/llm.tl:78-112):
// shapes fixed when the op is made, pointers taken from each launch's arguments.
struct RopeArgs {
  const int* pos = nullptr;
  const int* slot = nullptr;
  const float* Ct = nullptr;
  const float* St = nullptr;
  __half *Q = nullptr, *Kc = nullptr, *Vc = nullptr, *Kd = nullptr, *Vd = nullptr;
  int H = 0, G = 0, D = 0, NPOS = 0, NS = 0;
};

struct Op {
  Kind kind;
  std::string name;
  std::vector<std::vector<int64_t>> shapes;
  int n_args = 0;
  // Scratch owned by the op (global memory beyond inputs and outputs), sized
  // when the op is made so that a launch allocates nothing.
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  // Kernel-specific tuning chosen when the op is made.
  int p0 = 0, p1 = 0, p2 = 0, p3 = 0;
  // A scalar launch argument on its way into the kernel's parameters (linear_scatter: which inbox).
  int aux = 0;
  RopeArgs rope;
  // FP8 kinds: a launch's scale arrays (rows of X, rows of W, rows of Wu) on their way to the kernel.
  const float* q8[3] = {nullptr, nullptr, nullptr};
  std::vector<MapEntry> maps;

  // The cached maps for `key`, or null; `fresh` returns a slot to fill (the cache is emptied
  // when it has grown past a few hundred entries: operands that keep changing).
  const MapEntry* find_maps(const uint64_t key[4]) const {
    for (const MapEntry& e : maps)
      if (e.key[0] == key[0] && e.key[1] == key[1] && e.key[2] == key[2] && e.key[3] == key[3]) return &e;
    return nullptr;
  }
  MapEntry* fresh_maps(const uint64_t key[4]) {
    if (maps.size() >= 512) maps.clear();
    maps.emplace_back();
    for (int i = 0; i < 4; ++i) maps.back().key[i] = key[i];
    return &maps.back();
  }
};

struct Ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = true;
  std::string err;
  std::map<uint64_t, size_t> allocs;  // device pointer -> bytes, for bounds checks
  std::vector<Op> ops;
  std::unordered_map<std::string, int> op_by_key;
  std::vector<cudaGraphExec_t> graphs;
  std::vector<size_t> graph_nodes;  // kernels each recorded graph holds
  bool capturing = false;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  uint64_t launches = 0;
  // Device word the kernels raise when a bounded wait runs out: 0 = healthy.
  unsigned int* status = nullptr;
  // cuTensorMapEncodeTiled, resolved through the runtime (no link to libcuda).
  void* encode_tiled = nullptr;
  // Tensor-parallel communicator (NCCL, loaded at run time), or null.
  void* nccl_lib = nullptr;
  void* comm = nullptr;
  int rank = 0, nranks = 1;
  // Launch every kernel with programmatic dependent launch: the next kernel's blocks may become
  // resident (and run their set-up) while this one drains; each kernel waits for its
  // predecessor itself (griddepcontrol.wait) before it touches activations. TB200_PDL=0 turns it off.
  bool pdl = true;
  // Per-kernel profile (Gpu::profile of src/gpu.rs:38-42): when on, every launch waits for its
  // kernel and adds its device time under (phase, kernel).
  bool profiling = false;
  std::string phase;
  std::map<std::pair<std::string, std::string>, std::pair<uint64_t, double>> profile;
  std::vector<std::pair<std::pair<std::string, std::string>, std::pair<uint64_t, double>>> profile_sorted;
};

int fail(Ctx* c, const std::string& msg);
int cuda_fail(Ctx* c, cudaError_t e, const char* what);

#define TB_CUDA(c, ...)                                              \
  do {                                                               \
    cudaError_t e__ = (__VA_ARGS__);                                 \
    if (e__ != cudaSuccess) return cuda_fail((c), e__, #__VA_ARGS__); \
  } while (0)

// A tiled tensor map over a row-major array of `rank` dims (dims[0] innermost).
// strides_bytes[i] is the stride of dims[i+1]. Returns 0 on success.
int make_tensor_map(Ctx* c, CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz);

// ---- tensor-parallel exchange over peer memory (csrc/tp.cu, and the scatter epilogue of csrc/gemm.cu)
constexpr int TP_MAX = 8;

// Lives in device memory; written once by the host after the ranks exchanged IPC handles.
// Pointer arrays are indexed by rank; a rank's own entries are its local pointers.
//
// Row r of a step belongs to rank r % n. part[w][o] is owner o's INBOX w: f32
// [n sources][ceil(T / n) rows][dim], where source s's projection kernel stores its partial of
// owner o's rows (linear_scatter). stage[o] is rank o's landing area for the other owners'
// finished rows: 32-bit words, [T][dim / 2] of two halves of h, or [T][dim] of one f32 of x on
// the last call of a step. Inboxes and landing areas hold 0xffffffff in every word that is not
// waiting to be consumed (csrc/tp.cu).
struct TpTable {
  float* part[2][TP_MAX];
  unsigned int* stage[TP_MAX];
  float* x;             // this rank's residual stream
  __half* h;            // this rank's normalised activations
  unsigned int* trace;  // trace builds only (may be null): call counters and time stamps
  int rank, nranks;
};

// Launchers, one per kernel family. `a` holds the launch arguments as the C
// ABI received them: device pointers, or scalar bits in the low 32 bits.
int make_glue(Ctx* c, Op& op);
int launch_glue(Ctx* c, Op& op, const uint64_t* a);
int make_gemm(Ctx* c, Op& op);
int launch_gemm(Ctx* c, Op& op, const uint64_t* a);
int tune_gemm(Ctx* c, Op& op, const uint64_t* a, float* best_us);
int make_decode(Ctx* c, Op& op);
int launch_decode(Ctx* c, Op& op, const uint64_t* a);
int make_prefill(Ctx* c, Op& op);
int make_tp(Ctx* c, Op& op);
int launch_tp(Ctx* c, Op& op, const uint64_t* a);
size_t tp_table_bytes();
size_t tp_trace_bytes();
int tp_fill_table(void* out, size_t out_bytes, int rank, int nranks, const uint64_t* inbox0, const uint64_t* inbox1,
                  const uint64_t* landing, uint64_t x, uint64_t h, uint64_t trace);
int launch_prefill(Ctx* c, Op& op, const uint64_t* a);

// Launches `kern` on the context's stream, as a cluster of (cluster_x, 1, cluster_z) when that
// is more than one CTA.
template <class... KArgs, class... Args>
inline cudaError_t launch_kc(Ctx* c, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_x,
                             int cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c->stream;
  cudaLaunchAttribute at[2];
  int n = 0;
  if (cluster_x * cluster_z > 1) {
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = (unsigned)cluster_x;
    at[n].val.clusterDim.y = 1;
    at[n].val.clusterDim.z = (unsigned)cluster_z;
    ++n;
  }
  if (c->pdl) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = at;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// The common case: a cluster of (1, 1, cluster_z).
template <class... KArgs, class... Args>
inline cudaError_t launch_k(Ctx* c, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_z,
                            Args&&... args) {
  return launch_kc(c, kern, grid, block, smem, 1, cluster_z, static_cast<Args&&>(args)...);
}

inline float bits_f32(uint64_t v) {
  uint32_t u = (uint32_t)v;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

// ---------------------------------------------------------------------------
// Device side
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

// Waits give up after this many nanoseconds, raise the status word and let the
// kernel run to its end (results are then garbage, the context stays usable).
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

// Programmatic dependent launch. pdl_launch: the next kernel in the stream may start being
// scheduled. pdl_wait: everything the previous kernels wrote is complete and visible; every
// thread calls it before it reads or writes a buffer another kernel touches.
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on an mbarrier phase. On time-out the global status word gets
// `code` and every later wait of the grid returns at once.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* status, unsigned int code) {
  if (mbar_try(bar, parity)) return;
  const unsigned long long t0 = globaltimer();
  unsigned int spins = 0;
  while (!mbar_try(bar, parity)) {
    if ((++spins & 1023u) == 0) {
      if (*(volatile unsigned int*)status != 0) return;
      if (globaltimer() - t0 > WAIT_LIMIT_NS) {
        atomicCAS(status, 0u, code);
        return;
      }
    }
  }
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)m) : "memory");
}

// TMA tile loads into this CTA's shared memory, completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"((uint64_t)m), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"((uint64_t)m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z,
                                            int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(dst)),
      "l"((uint64_t)m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], f16 inputs, f32 accumulation, one CTA.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster whose ranks differ in bit 0 run one MMA of
// M = 256 together. Each holds 128 rows of A and half of B's rows in its own shared memory, at
// the same offsets; the even CTA issues the MMA; each gets its 128 rows of D in its own tensor
// memory. Tensor memory is allocated by the same warp of both CTAs.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot_in_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same on E4M3 operands (kind::f8f6f4: 32 bytes of K per instruction, where f16 has 16
// elements; the instruction descriptor's format fields are 0 for E4M3 as they are for f16).
__device__ __forceinline__ void umma_q8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at `bar`'s offset in every CTA of `cta_mask` (cluster ranks) once every
// MMA issued so far by this thread is done: the pair's ring slots are freed in both CTAs at once.
// (A barrier signal, not a data copy: no load of any kind is broadcast here.)
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(cta_mask)
               : "memory");
}
// A TMA tile load into THIS CTA's shared memory whose completion is counted on a barrier of the
// pair's even CTA (`bar_cluster_addr`: a shared::cluster address from cluster_map).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(smem_u32(dst)),
      "l"((uint64_t)m), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

// 32 lanes x 32 columns of f32 from TMEM: thread i of the warp gets lane
// (base lane + i), registers r[0..31] are consecutive columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// The reverse: 32 registers of each thread into 32 columns of its TMEM lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Eight columns at a time, for code that must stay small in registers.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M x 16 f16, one row per lane, two values per
// 32-bit column) is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor (sm_100 format, version 1), 128-byte swizzle.
// K-major tiles: rows of 128 bytes, 8-row groups `sbo` bytes apart.
// MN-major tiles: 64-element blocks `lbo` bytes apart, 8-k groups `sbo` apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: f16 A and B, f32 D, M x N tile.
// b_mn = 1 when B is stored N-major (a [K,N] row-major operand).
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N, int a_mn, int b_mn) {
  return (1u << 4)                      // D format f32
         | (0u << 7) | (0u << 10)       // A, B format f16
         | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---- thread-block clusters ------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Barrier over every thread of every CTA of the cluster; orders shared-memory
// accesses (local and remote) before it against those after it.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of `local` (a shared-memory address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Packs two f32 into f16x2 (round to nearest even), low half = a.
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

#endif  // __CUDACC__

}  // namespace tb
