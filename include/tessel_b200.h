/*
 * libtessel_b200 - C ABI.
 *
 * A drop-in for the launch path of the tessel LLM engine: everything
 * src/llm/engine.rs does on a device goes through `Gpu` (src/gpu.rs:28-263),
 * and each entry point below stands where one method of `Gpu` stands. The
 * kernels behind `tb200_kernel` are hand-written sm_100a CUDA, compiled ahead
 * of time; there is no JIT and no CPU path. All functions return 0 on success
 * and a non-zero code on failure, with the text (CUDA error number and string
 * included, as src/driver.rs:181-195 formats it) available from
 * `tb200_last_error`. Nothing throws or aborts across this boundary.
 *
 * One context drives one device on one stream, from one thread at a time
 * (the contract of src/runtime.rs:48-52). A tensor-parallel run is one process
 * and one context per GPU.
 *
 * Device memory is addressed by plain 64-bit device pointers; buffers from
 * `tb200_alloc` and buffers allocated elsewhere (another CUDA library in the
 * same process) are both accepted by every call.
 */
#ifndef TESSEL_B200_H
#define TESSEL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tb200_ctx tb200_ctx;
typedef int32_t tb200_op;    /* a kernel specialised for its shapes: `K` of src/gpu.rs:48 */
typedef int32_t tb200_graph; /* a recorded step: `GraphExec` of src/driver.rs */

/* Gpu::new (src/gpu.rs:53-67) + Cuda::new (src/driver.rs:150-175): binds
 * `device`, creates the stream. Fails if the device is not compute capability
 * 10.x. */
int tb200_init(int device, tb200_ctx** out);
void tb200_destroy(tb200_ctx* ctx);

/* The message of the last failed call on `ctx` (NULL: of the last failed
 * tb200_init). Valid until the next call on the same context. */
const char* tb200_last_error(tb200_ctx* ctx);

/* Gpu::alloc (src/gpu.rs:70-85): `bytes` of device memory, zero-filled. */
int tb200_alloc(tb200_ctx* ctx, size_t bytes, uint64_t* dptr);
/* The reference never frees (process lifetime); offered for long-lived hosts. */
int tb200_free(tb200_ctx* ctx, uint64_t dptr);

/* Gpu::write (src/gpu.rs:88-107): synchronous host-to-device copy at byte
 * `offset`; bounds-checked against the allocation when `dptr` came from
 * tb200_alloc. */
int tb200_write(tb200_ctx* ctx, uint64_t dptr, size_t offset, const void* src, size_t bytes);
/* Asynchronous variant on the context's stream; `src` must stay valid (and
 * should be pinned) until the next tb200_sync. */
int tb200_write_async(tb200_ctx* ctx, uint64_t dptr, size_t offset, const void* src, size_t bytes);

/* Gpu::read (src/gpu.rs:110-131): waits for the stream, then copies
 * device-to-host. */
int tb200_read(tb200_ctx* ctx, uint64_t dptr, size_t offset, void* dst, size_t bytes);

/* No counterpart in the reference (its host buffers are pageable Vec<u8>):
 * page-locked host memory, so that tb200_write_async / tb200_read move data at
 * full PCIe speed and asynchronously. */
int tb200_host_alloc(tb200_ctx* ctx, size_t bytes, void** out);
int tb200_host_free(tb200_ctx* ctx, void* ptr);

/* Gpu::kernel (src/gpu.rs:148-172): the kernel `name` for these array shapes,
 * made once and cached. `shapes` holds the dimensions of every array
 * parameter back to back, in the kernel's parameter order (kernels/llm.tl),
 * `ranks[i]` the number of dimensions of array i. Names: embed, rmsnorm,
 * linear, linear_residual, logits, gate_up, rope_q, kv_write,
 * prefill_attention, decode_attention, rmsnorm_rows (kernels/llm.tl:10-182),
 * matmul (kernels/matmul.tl:3-17), flash_attention, paged_attention
 * (kernels/attention.tl:4-51); and, with no counterpart in the reference,
 * linear_f32 (X[M,K], W[N,K], Y f32[M,N]), residual_add (R f32[M,N], P
 * f32[M,N]), argmax_rows (X f32[M,N], out i32[M]), rope_kv (rope_q and kv_write
 * in one launch: QKV, pos, slot, C, S, Q, Kc, Vc, K, V) and decode_advance
 * (picked[T], tok[T], pos[T], slot[T], lens[T], table[T,MP], hist[S,T], then
 * the i32 scalars n, P and step: the next decode step's inputs for rows < n,
 * computed on the device as src/llm/sched.rs:139-144 computes them on the
 * host, the picks also stored in hist[step]); argmax_partial (X f32[M,N],
 * pairs f32[R,M,2], then the i32 scalars rank and base: with the LM head's rows
 * split across R ranks, this rank's first maximum over its columns
 * [base, base+N) as (value, index) in slot `rank`, zeros in the other slots, so
 * that tb200_allreduce gathers the slots) and argmax_merge (pairs f32[R,M,2],
 * out i32[M]: the first maximum over the ranks, the token src/llm/mod.rs:132-140
 * picks from the whole row); and chunk_attention (Q[T,H,D], Kc[NP,P,G,D],
 * Vc[NP,P,G,D], table[T,MP], meta i32[C,4], O[T,H,D], then the f32 scale):
 * causal attention for the rows of prompts that are fed in pieces (the
 * reference needs a prompt to fit one step, src/llm/sched.rs:76-81). Chunk c
 * is rows [meta[c][0], meta[c][0] + meta[c][1]) of the step, the tokens at
 * positions meta[c][2], meta[c][2] + 1, ... of their sequence, whose block
 * table is row meta[c][0] of `table`; row r attends to cache positions 0 to
 * its own, this step's keys included (kv_write runs first). Rows outside every
 * chunk are not written.
 *
 * FP8 mode (no counterpart in the reference, which computes in f16; results
 * differ from the f16 kernels by the quantisation): E4M3 bytes with one f32
 * scale per row, value = decode(byte) * scale, scale = max|row| / 448 (1 for a
 * row of zeros), rounding to nearest even, saturating. quant_rows (X f16[M,K],
 * Q u8[M,K], S f32[M]; K a multiple of 8) quantises rows; rmsnorm_q8 (X
 * f32[T,Dm], W f16[Dm], Q u8[T,Dm], S f32[T], then the f32 eps) is rmsnorm
 * followed by quant_rows of its f16 result, in one launch. linear_q8 and
 * linear_residual_q8 (Xq u8[M,K], sx f32[M], Wq u8[N,K], sw f32[N], Y[M,N] f16
 * / f32 accumulated into) and gate_up_q8 (Xq, sx, Wgq, sg, Wuq, su, Y
 * f16[M,F]) are linear, linear_residual and gate_up on the 8-bit tensor-core
 * path with f32 accumulation, the product scaled by sx[row] * sw[column] before
 * the epilogue's own arithmetic; K a multiple of 16, N a multiple of 8.
 *
 * The reference's `meta` and `warps` arguments have no equivalent: tile shapes
 * are chosen inside. */
int tb200_kernel(tb200_ctx* ctx, const char* name, const int64_t* shapes, const int32_t* ranks, int n_arrays,
                 tb200_op* out);

/* Gpu::launch (src/gpu.rs:179-217): asynchronous launch on the context's
 * stream. `args[i]` is a device pointer for an array parameter, or the bits of
 * an f32/i32 scalar in the low 32 bits (src/gpu.rs:192-193), in the kernel's
 * parameter order.
 *
 * Kernels are launched with programmatic dependent launch: a kernel may start
 * while its predecessor on the stream drains, and waits for the predecessor
 * itself before it touches activations. The projections (linear,
 * linear_residual, logits, linear_f32, gate_up) request their first WEIGHT
 * tiles before that wait. So a weight operand W must be complete before the
 * previous kernel on the stream starts: weights written once at load time
 * satisfy this; a W produced on the stream by the kernel launched just before
 * (a dequantised or merged weight) does not, unless a tb200_sync or any other
 * kernel lies in between, or the process runs with TB200_PDL=0, which restores
 * plain stream order. matmul (both operands are activations) has no such
 * restriction. */
int tb200_launch(tb200_ctx* ctx, tb200_op op, const uint64_t* args, int n_args);

/* Engine::mm (src/llm/engine.rs:233-270), moved behind the boundary because the
 * tile shapes live here: the candidate tile configurations of a projection
 * kernel (linear, linear_residual, logits, linear_f32, gate_up, matmul) are
 * timed on the device, on `args` (the launch arguments of tb200_launch; the
 * kernel's output is overwritten, or for linear_residual accumulated into,
 * some tens of times: tune before the step that rewrites it, as the reference
 * does), with the L2 overwritten between launches, and the fastest is kept for
 * every later launch of `op`. `plan`, if not NULL, receives the choice as
 * {MT, BN, splits} (MT 3 = a CTA pair; zeros for a kernel with nothing to
 * choose), `best_us` its median time. Other kernels: nothing to tune, success.
 * Not during capture; allocates and frees a 192 MB scratch buffer (timing goes
 * on without the L2 overwrite if that allocation fails). With
 * TB200_GEMM_PLAN set in the environment the forced plan stays. */
int tb200_tune(tb200_ctx* ctx, tb200_op op, const uint64_t* args, int n_args, int32_t* plan, float* best_us);

/* Gpu::capture_begin / capture_end / replay (src/gpu.rs:233-247). */
int tb200_capture_begin(tb200_ctx* ctx);
int tb200_capture_end(tb200_ctx* ctx, tb200_graph* out);
int tb200_replay(tb200_ctx* ctx, tb200_graph graph);

/* Gpu::sync (src/gpu.rs:249-254). Also reports a kernel whose bounded wait
 * ran out since the last sync. */
int tb200_sync(tb200_ctx* ctx);

/* Cuda::time (src/driver.rs:366-380), split in two: events on the context's
 * stream around whatever is launched in between; `ms` is device time. */
int tb200_time_begin(tb200_ctx* ctx);
int tb200_time_end(tb200_ctx* ctx, float* ms);

/* Gpu::profile, Gpu::phase and Gpu::profile_rows (src/gpu.rs:38-42, :198-222).
 * tb200_profile(ctx, 1) clears the table and starts profiling: every
 * tb200_launch (and tb200_allreduce) then waits for its kernel and adds its
 * device time under (phase, kernel), where kernel is the name followed by the
 * shape of its last array, e.g. "linear -> [256, 6144]"; launches recorded into
 * a graph are not timed, so profile with plain launches. tb200_profile(ctx, 0)
 * stops it (the table stays). tb200_phase names the phase later launches are
 * counted under ("prefill", "decode"). tb200_profile_rows sorts the table,
 * largest total first, and returns the number of rows; tb200_profile_row reads
 * row i (strings valid until the next tb200_profile_rows or tb200_profile). */
int tb200_profile(tb200_ctx* ctx, int on);
int tb200_phase(tb200_ctx* ctx, const char* phase);
int tb200_profile_rows(tb200_ctx* ctx, int* n_rows);
int tb200_profile_row(tb200_ctx* ctx, int i, const char** phase, const char** kernel, uint64_t* launches, double* ms);

/* Gpu::launches (src/gpu.rs:37): kernels launched through this context
 * (a replayed graph counts every kernel it holds). */
int tb200_launch_count(tb200_ctx* ctx, uint64_t* out);

/* No counterpart in the reference: run on a stream the host already owns
 * (a `cudaStream_t`), so that other libraries' work can be ordered with the
 * kernels. NULL restores the context's own stream. */
int tb200_set_stream(tb200_ctx* ctx, void* cuda_stream);
/* The stream in use, as a `cudaStream_t`. */
int tb200_get_stream(tb200_ctx* ctx, void** cuda_stream);

/* Tensor parallelism (the reference has none: src/driver.rs:154 takes device
 * 0 only). One process per GPU: rank 0 obtains an id, the host hands it to the
 * other ranks, every rank joins, and tb200_allreduce sums `count` elements in
 * place across ranks on the context's stream (NCCL over NVLink). dtype: 0 =
 * f32, 1 = f16. */
#define TB200_COMM_ID_BYTES 128
int tb200_comm_id(tb200_ctx* ctx, void* id_out);
int tb200_comm_init(tb200_ctx* ctx, int rank, int nranks, const void* id);
int tb200_allreduce(tb200_ctx* ctx, uint64_t dptr, size_t count, int dtype);

/* No counterpart in the reference: the cross-rank sum fused with the residual add
 * and the next RMSNorm, over peer memory (NVLink stores; every wait polls local
 * memory) instead of an NCCL call. Row r of a step belongs to rank r % nranks.
 * Each rank allocates two inboxes f32[nranks][ceil(T/nranks)][dim] (allocate
 * (T + nranks) * dim * 4 bytes each) and a landing area of T*dim*4 bytes (where
 * the other owners' finished rows arrive), FILLS ALL THREE WITH 0xff BYTES
 * (tb200_memset) - the 32-bit pattern 0xffffffff marks a word that holds
 * nothing; the kernels wait for a word to differ from it, and put it back into
 * every word they have consumed, so the fill is needed once - and exports them
 * with tb200_ipc_export (a 64-byte handle each); the host hands every rank the
 * others' handles, tb200_ipc_import maps them, and tb200_tp_table writes the
 * table (`inbox0`, `inbox1`, `landing`: arrays indexed by rank, a rank's own
 * entry its local pointer; `x` f32[T,dim] and `h` f16[T,dim]: this rank's own
 * residual stream and normalised activations; `trace`: 0, or for a trace build
 * of the library a zero-filled buffer of tb200_tp_sizes' trace size) that the
 * host then uploads to device memory.
 *
 * The kernel "linear_scatter" (arrays: X f16[M,K], W f16[N,K], table u8[bytes];
 * then which i32) is linear_f32 whose output row r is stored into inbox `which`
 * of rank r % nranks, at [this rank][r / nranks] - the reduce-scatter, done by
 * the projection itself. The kernel "tp_reduce_norm" (arrays: table u8[bytes],
 * W f16[dim], X f32[T,dim]; then eps f32, which i32 = the inbox to sum, do_norm
 * i32, nranks i32) runs behind it: for each row this rank owns it waits until
 * the nranks partials have arrived in its inbox, adds them, in rank order, to x
 * and, if do_norm, normalises the row into h; it sends the rows to every peer
 * and collects the peers', which leaves h identical on every rank (x is then
 * current only in the rows this rank owns); with do_norm = 0 it leaves x
 * identical on every rank instead. Every rank must launch both the same number
 * of times with the same shapes, and consecutive pairs must alternate `which`
 * (a rank may write into an inbox again only after the call that read it and
 * one more have passed: the alternation guarantees it). A wait that does not
 * end within a second raises the status word (401: partials, 402: rows) and the
 * kernel returns; the exchange buffers are then in an undefined state. */
#define TB200_IPC_HANDLE_BYTES 64
int tb200_ipc_export(tb200_ctx* ctx, uint64_t dptr, void* handle);
int tb200_ipc_import(tb200_ctx* ctx, const void* handle, uint64_t* dptr);
int tb200_tp_sizes(size_t* table_bytes, size_t* trace_bytes);
int tb200_tp_table(tb200_ctx* ctx, void* host_out, size_t bytes, int rank, int nranks, const uint64_t* inbox0,
                   const uint64_t* inbox1, const uint64_t* landing, uint64_t x, uint64_t h, uint64_t trace);
/* Fills `bytes` bytes at `dptr` with the byte `value`, on the context's stream;
 * bounds-checked like tb200_write. */
int tb200_memset(tb200_ctx* ctx, uint64_t dptr, int value, size_t bytes);

/* No counterpart in the reference. Paged decode attention (the computation of
 * the "decode_attention" kernel above) for callers that cannot allocate device
 * memory: a host that gave its whole device-memory budget to its own pool at
 * start-up, or that must not enter the allocator where it runs. The kernel's
 * split-KV scratch is a 16 MiB array inside the library image (held by every
 * GPU that loads the library, until the process exits) instead of an
 * allocation; this call performs no cudaMalloc / cudaFree.
 *   dims = {B, H, G, D, NP, P, MP}: Q, O f16 [B,H,D]; Kc, Vc f16 [NP,P,G,D];
 *   table i32 [B,MP]; lens i32 [B].
 * Limit: B*H*(D+2)*4 bytes (one split's partials) must fit the 16 MiB, else the
 * call fails with a message saying so; within the limit the number of KV
 * splits is reduced to what fits. The first call on a device resolves the
 * array's device address and sets kernel attributes: make that first call
 * before any stream capture. All calls on a device share the one array and it
 * keeps the previous call's contents (nothing in it has to be cleared); two
 * calls that overlap on the GPU (different streams or contexts) would race on
 * it, so keep them on one stream. */
int tb200_decode_attention_static(tb200_ctx* ctx, const int32_t* dims, uint64_t q, uint64_t kc, uint64_t vc,
                                  uint64_t table, uint64_t lens, uint64_t o, float scale);

/* Host helper: the seeded xorshift generator of src/bench.rs:13-35, as
 * Weights::random (src/llm/mod.rs:80-108) draws from it. `state` starts as
 * tb200_rng_seed(seed). */
uint64_t tb200_rng_seed(uint64_t seed);
void tb200_rng_uniform(uint64_t* state, float* out, size_t n);

#ifdef __cplusplus
}
#endif
#endif /* TESSEL_B200_H */
