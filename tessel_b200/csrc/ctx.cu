// The C ABI of libtessel_b200 (include/tessel_b200.h): context, buffers, the
// op table, graphs, timing, and the tensor-parallel communicator.
#include <dlfcn.h>
#include <string.h>

#include <algorithm>
#include <sstream>

#include "../../include/tessel_b200.h"
#include "common.cuh"

struct tb200_ctx {
  tb::Ctx c;
};

namespace tb {

static std::string g_init_error;

int fail(Ctx* c, const std::string& msg) {
  if (c)
    c->err = msg;
  else
    g_init_error = msg;
  return 1;
}

int cuda_fail(Ctx* c, cudaError_t e, const char* what) {
  std::ostringstream s;
  s << what << ": CUDA error " << (int)e << " (" << cudaGetErrorString(e) << ")";
  // A failed launch leaves a sticky "last error"; clear it so the next call reports its own.
  cudaGetLastError();
  return fail(c, s.str());
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tensor_map(Ctx* c, CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  CUresult r = ((EncodeTiled)c->encode_tiled)(out, dt, (cuuint32_t)rank, const_cast<void*>(base),
                                               (const cuuint64_t*)dims, (const cuuint64_t*)strides_bytes,
                                               (const cuuint32_t*)box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::ostringstream s;
    s << "cuTensorMapEncodeTiled failed with " << (int)r << " (rank " << rank << ", dims";
    for (int i = 0; i < rank; ++i) s << " " << dims[i];
    s << ", box";
    for (int i = 0; i < rank; ++i) s << " " << box[i];
    s << ", base " << base << ")";
    return fail(c, s.str());
  }
  return 0;
}

struct KindInfo {
  const char* name;
  Kind kind;
  int n_arrays;
  int n_args;
};

static const KindInfo KINDS[] = {
    {"embed", K_EMBED, 3, 3},
    {"rmsnorm", K_RMSNORM, 3, 4},
    {"linear", K_LINEAR, 3, 3},
    {"linear_residual", K_LINEAR_RESIDUAL, 3, 3},
    {"logits", K_LOGITS, 3, 3},
    {"gate_up", K_GATE_UP, 4, 4},
    {"rope_q", K_ROPE_Q, 5, 5},
    {"kv_write", K_KV_WRITE, 9, 9},
    {"prefill_attention", K_PREFILL_ATTENTION, 5, 6},
    {"decode_attention", K_DECODE_ATTENTION, 6, 7},
    {"rmsnorm_rows", K_RMSNORM_ROWS, 4, 5},
    {"matmul", K_MATMUL, 3, 3},
    {"flash_attention", K_FLASH_ATTENTION, 4, 5},
    {"paged_attention", K_PAGED_ATTENTION, 6, 7},
    {"linear_f32", K_LINEAR_F32, 3, 3},
    {"residual_add", K_RESIDUAL_ADD, 2, 2},
    {"argmax_rows", K_ARGMAX_ROWS, 2, 2},
    {"decode_advance", K_DECODE_ADVANCE, 7, 10},
    {"tp_reduce_norm", K_TP_REDUCE_NORM, 3, 7},
    {"rope_kv", K_ROPE_KV, 10, 10},
    {"argmax_partial", K_ARGMAX_PARTIAL, 2, 4},
    {"argmax_merge", K_ARGMAX_MERGE, 2, 2},
    {"chunk_attention", K_CHUNK_ATTENTION, 6, 7},
    {"linear_scatter", K_LINEAR_SCATTER, 3, 4},
    {"linear_rope_kv", K_LINEAR_ROPE_KV, 12, 12},
    {"quant_rows", K_QUANT_ROWS, 3, 3},
    {"rmsnorm_q8", K_RMSNORM_Q8, 4, 5},
    {"linear_q8", K_LINEAR_Q8, 5, 5},
    {"linear_residual_q8", K_LINEAR_RESIDUAL_Q8, 5, 5},
    {"gate_up_q8", K_GATE_UP_Q8, 7, 7},
};

static std::string shape_text(const std::vector<int64_t>& s) {
  std::ostringstream o;
  o << "[";
  for (size_t i = 0; i < s.size(); ++i) o << (i ? ", " : "") << s[i];
  o << "]";
  return o.str();
}

// Closes the event pair opened before a profiled launch and books its time under (phase, kernel).
static int profile_add(Ctx* c, const std::string& kernel) {
  float ms = 0.f;
  TB_CUDA(c, cudaEventRecord(c->ev1, c->stream));
  TB_CUDA(c, cudaEventSynchronize(c->ev1));
  TB_CUDA(c, cudaEventElapsedTime(&ms, c->ev0, c->ev1));
  auto& e = c->profile[{c->phase, kernel}];
  e.first += 1;
  e.second += ms;
  return 0;
}

static bool is_gemm(Kind k) {
  return k == K_LINEAR || k == K_LINEAR_RESIDUAL || k == K_LOGITS || k == K_GATE_UP || k == K_MATMUL ||
         k == K_LINEAR_F32 || k == K_LINEAR_SCATTER || k == K_LINEAR_ROPE_KV || k == K_LINEAR_Q8 ||
         k == K_LINEAR_RESIDUAL_Q8 || k == K_GATE_UP_Q8;
}

}  // namespace tb

using namespace tb;

extern "C" {

int tb200_init(int device, tb200_ctx** out) {
  if (!out) return fail(nullptr, "tb200_init: out is NULL");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceCount");
  if (device < 0 || device >= n) {
    std::ostringstream s;
    s << "tb200_init: device " << device << " of " << n;
    return fail(nullptr, s.str());
  }
  cudaDeviceProp p;
  e = cudaGetDeviceProperties(&p, device);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceProperties");
  if (p.major != 10) {
    std::ostringstream s;
    s << "tb200_init: device " << device << " is compute capability " << p.major << "." << p.minor
      << "; this library holds sm_100a code only";
    return fail(nullptr, s.str());
  }
  e = cudaSetDevice(device);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaSetDevice");
  tb200_ctx* h = new tb200_ctx();
  Ctx* c = &h->c;
  c->device = device;
  c->sm_count = p.multiProcessorCount;
  if (const char* e = getenv("TB200_PDL")) c->pdl = atoi(e) != 0;
  auto bail = [&](cudaError_t er, const char* what) {
    cuda_fail(nullptr, er, what);
    delete h;
    return 1;
  };
  if ((e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking)) != cudaSuccess)
    return bail(e, "cudaStreamCreate");
  if ((e = cudaEventCreate(&c->ev0)) != cudaSuccess) return bail(e, "cudaEventCreate");
  if ((e = cudaEventCreate(&c->ev1)) != cudaSuccess) return bail(e, "cudaEventCreate");
  if ((e = cudaMalloc((void**)&c->status, 256)) != cudaSuccess) return bail(e, "cudaMalloc(status)");
  if ((e = cudaMemset(c->status, 0, 256)) != cudaSuccess) return bail(e, "cudaMemset(status)");
  cudaDriverEntryPointQueryResult q;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &c->encode_tiled, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !c->encode_tiled)
    return bail(e == cudaSuccess ? cudaErrorUnknown : e, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
  *out = h;
  return 0;
}

void tb200_destroy(tb200_ctx* h) {
  if (!h) return;
  Ctx* c = &h->c;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (auto g : c->graphs)
    if (g) cudaGraphExecDestroy(g);
  for (auto& op : c->ops)
    if (op.scratch) cudaFree(op.scratch);
  for (auto& a : c->allocs) cudaFree((void*)a.first);
  if (c->status) cudaFree(c->status);
  if (c->ev0) cudaEventDestroy(c->ev0);
  if (c->ev1) cudaEventDestroy(c->ev1);
  if (c->own_stream && c->stream) cudaStreamDestroy(c->stream);
  if (c->comm && c->nccl_lib) {
    typedef int (*Destroy)(void*);
    Destroy d = (Destroy)dlsym(c->nccl_lib, "ncclCommDestroy");
    if (d) d(c->comm);
  }
  delete h;
}

const char* tb200_last_error(tb200_ctx* h) { return h ? h->c.err.c_str() : g_init_error.c_str(); }

int tb200_alloc(tb200_ctx* h, size_t bytes, uint64_t* dptr) {
  Ctx* c = &h->c;
  if (!dptr) return fail(c, "tb200_alloc: dptr is NULL");
  size_t free_b = 0, total_b = 0;
  TB_CUDA(c, cudaSetDevice(c->device));
  TB_CUDA(c, cudaMemGetInfo(&free_b, &total_b));
  if (bytes > free_b) {
    // Refused before the allocator is asked, so an oversized request cannot disturb the device.
    std::ostringstream s;
    s << "tb200_alloc: " << bytes << " bytes requested, " << free_b << " free of " << total_b;
    return fail(c, s.str());
  }
  void* p = nullptr;
  TB_CUDA(c, cudaMalloc(&p, bytes ? bytes : 1));
  cudaError_t e = cudaMemsetAsync(p, 0, bytes, c->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(c, e, "cudaMemset");
  }
  c->allocs[(uint64_t)p] = bytes;
  *dptr = (uint64_t)p;
  return 0;
}

int tb200_free(tb200_ctx* h, uint64_t dptr) {
  Ctx* c = &h->c;
  auto it = c->allocs.find(dptr);
  if (it == c->allocs.end()) return fail(c, "tb200_free: not a pointer tb200_alloc returned");
  TB_CUDA(c, cudaStreamSynchronize(c->stream));
  TB_CUDA(c, cudaFree((void*)dptr));
  c->allocs.erase(it);
  return 0;
}

// Bounds check against the owning allocation, when there is one.
static int check_range(Ctx* c, const char* what, uint64_t dptr, size_t offset, size_t bytes) {
  auto it = c->allocs.upper_bound(dptr);
  if (it == c->allocs.begin()) return 0;
  --it;
  if (dptr >= it->first + (it->second ? it->second : 1)) return 0;  // foreign pointer
  const size_t base_off = (size_t)(dptr - it->first);
  if (base_off + offset + bytes > it->second) {
    std::ostringstream s;
    s << what << " of " << bytes << " bytes at " << (base_off + offset) << " in a buffer of " << it->second;
    return fail(c, s.str());
  }
  return 0;
}

int tb200_write(tb200_ctx* h, uint64_t dptr, size_t offset, const void* src, size_t bytes) {
  Ctx* c = &h->c;
  if (check_range(c, "write", dptr, offset, bytes)) return 1;
  if (bytes == 0) return 0;
  TB_CUDA(c, cudaMemcpyAsync((void*)(dptr + offset), src, bytes, cudaMemcpyHostToDevice, c->stream));
  if (!c->capturing) TB_CUDA(c, cudaStreamSynchronize(c->stream));
  return 0;
}

int tb200_write_async(tb200_ctx* h, uint64_t dptr, size_t offset, const void* src, size_t bytes) {
  Ctx* c = &h->c;
  if (check_range(c, "write", dptr, offset, bytes)) return 1;
  if (bytes == 0) return 0;
  TB_CUDA(c, cudaMemcpyAsync((void*)(dptr + offset), src, bytes, cudaMemcpyHostToDevice, c->stream));
  return 0;
}

int tb200_read(tb200_ctx* h, uint64_t dptr, size_t offset, void* dst, size_t bytes) {
  Ctx* c = &h->c;
  if (check_range(c, "read", dptr, offset, bytes)) return 1;
  if (c->capturing) return fail(c, "tb200_read during graph capture");
  if (bytes)
    TB_CUDA(c, cudaMemcpyAsync(dst, (const void*)(dptr + offset), bytes, cudaMemcpyDeviceToHost, c->stream));
  return tb200_sync(h);
}

int tb200_host_alloc(tb200_ctx* h, size_t bytes, void** out) {
  Ctx* c = &h->c;
  if (!out) return fail(c, "tb200_host_alloc: out is NULL");
  TB_CUDA(c, cudaSetDevice(c->device));
  TB_CUDA(c, cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
  return 0;
}

int tb200_host_free(tb200_ctx* h, void* ptr) {
  Ctx* c = &h->c;
  TB_CUDA(c, cudaFreeHost(ptr));
  return 0;
}

int tb200_kernel(tb200_ctx* h, const char* name, const int64_t* shapes, const int32_t* ranks, int n_arrays,
                 tb200_op* out) {
  Ctx* c = &h->c;
  if (!name || !out || (n_arrays > 0 && (!shapes || !ranks))) return fail(c, "tb200_kernel: NULL argument");
  const KindInfo* info = nullptr;
  for (const KindInfo& k : KINDS)
    if (!strcmp(k.name, name)) info = &k;
  if (!info) return fail(c, std::string("no kernel ") + name);
  if (n_arrays != info->n_arrays) {
    std::ostringstream s;
    s << name << " takes " << info->n_arrays << " arrays, " << n_arrays << " shapes given";
    return fail(c, s.str());
  }
  std::ostringstream key;
  key << name;
  Op op;
  op.kind = info->kind;
  op.name = name;
  op.n_args = info->n_args;
  const int64_t* p = shapes;
  for (int i = 0; i < n_arrays; ++i) {
    if (ranks[i] < 1 || ranks[i] > 4) return fail(c, std::string(name) + ": array ranks are 1 to 4");
    std::vector<int64_t> s(p, p + ranks[i]);
    key << " [";
    for (int64_t d : s) {
      if (d < 0) return fail(c, std::string(name) + ": negative dimension");
      key << d << ",";
    }
    key << "]";
    op.shapes.push_back(s);
    p += ranks[i];
  }
  auto it = c->op_by_key.find(key.str());
  if (it != c->op_by_key.end()) {
    *out = it->second;
    return 0;
  }
  TB_CUDA(c, cudaSetDevice(c->device));
  int r;
  if (is_gemm(op.kind))
    r = make_gemm(c, op);
  else if (op.kind == K_DECODE_ATTENTION || op.kind == K_PAGED_ATTENTION)
    r = make_decode(c, op);
  else if (op.kind == K_PREFILL_ATTENTION || op.kind == K_FLASH_ATTENTION || op.kind == K_CHUNK_ATTENTION)
    r = make_prefill(c, op);
  else if (op.kind == K_TP_REDUCE_NORM)
    r = make_tp(c, op);
  else
    r = make_glue(c, op);
  if (r) return r;
  c->ops.push_back(op);
  *out = (tb200_op)(c->ops.size() - 1);
  c->op_by_key[key.str()] = *out;
  return 0;
}

int tb200_launch(tb200_ctx* h, tb200_op id, const uint64_t* args, int n_args) {
  Ctx* c = &h->c;
  if (id < 0 || (size_t)id >= c->ops.size()) return fail(c, "tb200_launch: no such kernel handle");
  Op& op = c->ops[id];
  if (n_args != op.n_args) {
    std::ostringstream s;
    s << op.name << " takes " << op.n_args << " arguments, " << n_args << " given";
    return fail(c, s.str());
  }
  if (!args) return fail(c, "tb200_launch: args is NULL");
  const bool timed = c->profiling && !c->capturing;
  if (timed) TB_CUDA(c, cudaEventRecord(c->ev0, c->stream));
  int r;
  if (is_gemm(op.kind))
    r = launch_gemm(c, op, args);
  else if (op.kind == K_DECODE_ATTENTION || op.kind == K_PAGED_ATTENTION)
    r = launch_decode(c, op, args);
  else if (op.kind == K_PREFILL_ATTENTION || op.kind == K_FLASH_ATTENTION || op.kind == K_CHUNK_ATTENTION)
    r = launch_prefill(c, op, args);
  else if (op.kind == K_TP_REDUCE_NORM)
    r = launch_tp(c, op, args);
  else
    r = launch_glue(c, op, args);
  if (r || !timed) return r;
  return profile_add(c, op.name + " -> " + shape_text(op.shapes.empty() ? std::vector<int64_t>() : op.shapes.back()));
}

int tb200_tune(tb200_ctx* h, tb200_op id, const uint64_t* args, int n_args, int32_t* plan, float* best_us) {
  Ctx* c = &h->c;
  if (id < 0 || (size_t)id >= c->ops.size()) return fail(c, "tb200_tune: no such kernel handle");
  Op& op = c->ops[id];
  if (n_args != op.n_args || !args) return fail(c, op.name + ": tb200_tune takes the kernel's launch arguments");
  if (best_us) *best_us = 0.f;
  int r = 0;
  if (is_gemm(op.kind)) {
    TB_CUDA(c, cudaSetDevice(c->device));
    r = tune_gemm(c, op, args, best_us);
  }
  if (plan) {
    plan[0] = is_gemm(op.kind) && op.p0 == 1 ? op.p1 : 0;
    plan[1] = is_gemm(op.kind) && op.p0 == 1 ? op.p2 : 0;
    plan[2] = is_gemm(op.kind) && op.p0 == 1 ? op.p3 : 0;
  }
  return r;
}

int tb200_capture_begin(tb200_ctx* h) {
  Ctx* c = &h->c;
  if (c->capturing) return fail(c, "capture already begun");
  TB_CUDA(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeRelaxed));
  c->capturing = true;
  return 0;
}

int tb200_capture_end(tb200_ctx* h, tb200_graph* out) {
  Ctx* c = &h->c;
  if (!c->capturing) return fail(c, "capture_end without capture_begin");
  c->capturing = false;
  cudaGraph_t g = nullptr;
  TB_CUDA(c, cudaStreamEndCapture(c->stream, &g));
  cudaGraphExec_t x = nullptr;
  cudaError_t e = cudaGraphInstantiate(&x, g, 0);
  size_t nodes = 0;
  cudaGraphGetNodes(g, nullptr, &nodes);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return cuda_fail(c, e, "cudaGraphInstantiate");
  c->graphs.push_back(x);
  c->graph_nodes.push_back(nodes);
  if (out) *out = (tb200_graph)(c->graphs.size() - 1);
  return 0;
}

int tb200_replay(tb200_ctx* h, tb200_graph g) {
  Ctx* c = &h->c;
  if (g < 0 || (size_t)g >= c->graphs.size()) return fail(c, "tb200_replay: no such graph");
  TB_CUDA(c, cudaGraphLaunch(c->graphs[g], c->stream));
  c->launches += c->graph_nodes[g];
  return 0;
}

int tb200_sync(tb200_ctx* h) {
  Ctx* c = &h->c;
  TB_CUDA(c, cudaStreamSynchronize(c->stream));
  unsigned int st = 0;
  TB_CUDA(c, cudaMemcpy(&st, c->status, 4, cudaMemcpyDeviceToHost));
  if (st != 0) {
    cudaMemset(c->status, 0, 4);
    std::ostringstream s;
    s << "a kernel gave up a bounded wait (status " << st << "); its results are invalid";
    return fail(c, s.str());
  }
  return 0;
}

int tb200_time_begin(tb200_ctx* h) {
  Ctx* c = &h->c;
  TB_CUDA(c, cudaEventRecord(c->ev0, c->stream));
  return 0;
}

int tb200_time_end(tb200_ctx* h, float* ms) {
  Ctx* c = &h->c;
  TB_CUDA(c, cudaEventRecord(c->ev1, c->stream));
  TB_CUDA(c, cudaEventSynchronize(c->ev1));
  TB_CUDA(c, cudaEventElapsedTime(ms, c->ev0, c->ev1));
  return 0;
}

int tb200_profile(tb200_ctx* h, int on) {
  Ctx* c = &h->c;
  if (c->capturing) return fail(c, "tb200_profile during capture");
  if (on) {
    c->profile.clear();
    c->profile_sorted.clear();
  }
  c->profiling = on != 0;
  return 0;
}

int tb200_phase(tb200_ctx* h, const char* phase) {
  h->c.phase = phase ? phase : "";
  return 0;
}

int tb200_profile_rows(tb200_ctx* h, int* n_rows) {
  Ctx* c = &h->c;
  c->profile_sorted.assign(c->profile.begin(), c->profile.end());
  std::stable_sort(c->profile_sorted.begin(), c->profile_sorted.end(),
                   [](const auto& a, const auto& b) { return a.second.second > b.second.second; });
  if (n_rows) *n_rows = (int)c->profile_sorted.size();
  return 0;
}

int tb200_profile_row(tb200_ctx* h, int i, const char** phase, const char** kernel, uint64_t* launches, double* ms) {
  Ctx* c = &h->c;
  if (i < 0 || (size_t)i >= c->profile_sorted.size()) return fail(c, "tb200_profile_row: no such row (call tb200_profile_rows first)");
  const auto& r = c->profile_sorted[i];
  if (phase) *phase = r.first.first.c_str();
  if (kernel) *kernel = r.first.second.c_str();
  if (launches) *launches = r.second.first;
  if (ms) *ms = r.second.second;
  return 0;
}

int tb200_launch_count(tb200_ctx* h, uint64_t* out) {
  *out = h->c.launches;
  return 0;
}

int tb200_set_stream(tb200_ctx* h, void* s) {
  Ctx* c = &h->c;
  if (c->capturing) return fail(c, "tb200_set_stream during capture");
  if (s == nullptr) {
    if (!c->own_stream) {
      TB_CUDA(c, cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
      c->own_stream = true;
    }
    return 0;
  }
  if (c->own_stream && c->stream) {
    TB_CUDA(c, cudaStreamSynchronize(c->stream));
    cudaStreamDestroy(c->stream);
  }
  c->stream = (cudaStream_t)s;
  c->own_stream = false;
  return 0;
}

int tb200_get_stream(tb200_ctx* h, void** s) {
  *s = (void*)h->c.stream;
  return 0;
}

// ---- NCCL, bound at run time -------------------------------------------------
struct NcclId {
  char internal[TB200_COMM_ID_BYTES];
};
typedef int (*NcclGetUniqueId)(NcclId*);
typedef int (*NcclCommInitRank)(void**, int, NcclId, int);
typedef int (*NcclAllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef const char* (*NcclGetErrorString)(int);

static int nccl_open(Ctx* c) {
  if (c->nccl_lib) return 0;
  const char* names[] = {getenv("TB200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (!n) continue;
    c->nccl_lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (c->nccl_lib) return 0;
  }
  return fail(c, std::string("cannot load NCCL (set TB200_NCCL_LIB): ") + dlerror());
}

static int nccl_fail(Ctx* c, int code, const char* what) {
  NcclGetErrorString es = (NcclGetErrorString)dlsym(c->nccl_lib, "ncclGetErrorString");
  std::ostringstream s;
  s << what << ": NCCL error " << code << " (" << (es ? es(code) : "?") << ")";
  return fail(c, s.str());
}

int tb200_comm_id(tb200_ctx* h, void* id_out) {
  Ctx* c = &h->c;
  if (nccl_open(c)) return 1;
  NcclGetUniqueId f = (NcclGetUniqueId)dlsym(c->nccl_lib, "ncclGetUniqueId");
  if (!f) return fail(c, "ncclGetUniqueId not found");
  int r = f((NcclId*)id_out);
  return r ? nccl_fail(c, r, "ncclGetUniqueId") : 0;
}

int tb200_comm_init(tb200_ctx* h, int rank, int nranks, const void* id) {
  Ctx* c = &h->c;
  if (nranks < 1 || rank < 0 || rank >= nranks) return fail(c, "tb200_comm_init: bad rank");
  if (nccl_open(c)) return 1;
  NcclCommInitRank f = (NcclCommInitRank)dlsym(c->nccl_lib, "ncclCommInitRank");
  if (!f) return fail(c, "ncclCommInitRank not found");
  TB_CUDA(c, cudaSetDevice(c->device));
  NcclId nid;
  memcpy(&nid, id, sizeof nid);
  int r = f(&c->comm, nranks, nid, rank);
  if (r) return nccl_fail(c, r, "ncclCommInitRank");
  c->rank = rank;
  c->nranks = nranks;
  return 0;
}

int tb200_allreduce(tb200_ctx* h, uint64_t dptr, size_t count, int dtype) {
  Ctx* c = &h->c;
  if (c->nranks == 1 && !c->comm) return 0;  // a single rank owns the whole sum
  if (!c->comm) return fail(c, "tb200_allreduce before tb200_comm_init");
  if (dtype != 0 && dtype != 1) return fail(c, "tb200_allreduce: dtype is 0 (f32) or 1 (f16)");
  NcclAllReduce f = (NcclAllReduce)dlsym(c->nccl_lib, "ncclAllReduce");
  if (!f) return fail(c, "ncclAllReduce not found");
  const int nccl_f32 = 7, nccl_f16 = 6, nccl_sum = 0;
  const bool timed = c->profiling && !c->capturing;
  if (timed) TB_CUDA(c, cudaEventRecord(c->ev0, c->stream));
  int r = f((const void*)dptr, (void*)dptr, count, dtype == 0 ? nccl_f32 : nccl_f16, nccl_sum, c->comm, c->stream);
  if (r) return nccl_fail(c, r, "ncclAllReduce");
  c->launches += 1;
  if (timed) {
    std::ostringstream o;
    o << "allreduce -> [" << count << "]";
    return profile_add(c, o.str());
  }
  return 0;
}

int tb200_ipc_export(tb200_ctx* h, uint64_t dptr, void* handle) {
  Ctx* c = &h->c;
  static_assert(sizeof(cudaIpcMemHandle_t) == TB200_IPC_HANDLE_BYTES, "IPC handle size");
  TB_CUDA(c, cudaSetDevice(c->device));
  TB_CUDA(c, cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle, (void*)dptr));
  return 0;
}

int tb200_ipc_import(tb200_ctx* h, const void* handle, uint64_t* dptr) {
  Ctx* c = &h->c;
  TB_CUDA(c, cudaSetDevice(c->device));
  cudaIpcMemHandle_t hd;
  memcpy(&hd, handle, sizeof hd);
  void* p = nullptr;
  TB_CUDA(c, cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess));
  *dptr = (uint64_t)p;
  return 0;
}

int tb200_tp_sizes(size_t* table_bytes, size_t* trace_bytes) {
  if (table_bytes) *table_bytes = tp_table_bytes();
  if (trace_bytes) *trace_bytes = tp_trace_bytes();
  return 0;
}

int tb200_tp_table(tb200_ctx* h, void* out, size_t bytes, int rank, int nranks, const uint64_t* inbox0,
                   const uint64_t* inbox1, const uint64_t* landing, uint64_t x, uint64_t hh, uint64_t trace) {
  Ctx* c = &h->c;
  if (tp_fill_table(out, bytes, rank, nranks, inbox0, inbox1, landing, x, hh, trace))
    return fail(c, "tb200_tp_table: 1 to 8 ranks, rank inside, and a buffer of tb200_tp_sizes' table size");
  return 0;
}

int tb200_memset(tb200_ctx* h, uint64_t dptr, int value, size_t bytes) {
  Ctx* c = &h->c;
  if (c->capturing) return fail(c, "tb200_memset during graph capture");
  if (check_range(c, "memset", dptr, 0, bytes)) return 1;
  if (bytes == 0) return 0;
  TB_CUDA(c, cudaSetDevice(c->device));
  TB_CUDA(c, cudaMemsetAsync((void*)dptr, value, bytes, c->stream));
  return 0;
}

uint64_t tb200_rng_seed(uint64_t seed) { return (seed * 0x9e3779b97f4a7c15ull) | 1ull; }

void tb200_rng_uniform(uint64_t* state, float* out, size_t n) {
  uint64_t s = *state;
  for (size_t i = 0; i < n; ++i) {
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    out[i] = ((float)(s >> 40) / 16777216.0f) * 2.0f - 1.0f;
  }
  *state = s;
}

}  // extern "C"
