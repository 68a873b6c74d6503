/*
 * tvb200: C ABI of the B200 runtime and kernels behind torch-vulkan's
 * quantised matrix products.
 *
 * This is the boundary a host runtime binds (cgo / Rust FFI / ctypes / the
 * C++ ATen layer in torch_vulkan_b200/csrc/aten): plain pointers and sizes, no
 * torch types. It takes the place of the reference's C ABI between its C++
 * ATen layer and its Rust runtime (crates/pyvk/csrc/vk.h:49-69, implemented in
 * crates/pyvk/src/ffi.rs), with two changes: every call names a device (the
 * reference has one), and the stringly-typed vkt_dispatch(name, spec, push,
 * grid) is replaced by one typed launcher per kernel family.
 *
 * Conventions (as ffi.rs:1-4): functions return 0 on success and -1 on
 * failure, with the message available from tvb_last_error() on the same
 * thread. Kernels are queued on the device's stream (tvb_stream) and run
 * asynchronously; tvb_synchronize waits. All pointers passed to the kernel
 * launchers are device pointers unless said otherwise. There is no CPU
 * fallback anywhere: without a usable GPU every call fails with a message.
 */
#ifndef TVB200_H
#define TVB200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define TVB_API __attribute__((visibility("default")))
#else
#define TVB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Element types (the kernel-name suffixes of the reference: "f32", "f16", "bf16", ...). */
enum TvbDtype {
  TVB_F32 = 0,
  TVB_F16 = 1,
  TVB_BF16 = 2,
  TVB_E4M3 = 3, /* float8_e4m3fn */
  TVB_E5M2 = 4, /* float8_e5m2 */
  TVB_I8 = 5,
  TVB_U8 = 6,
  TVB_I32 = 7,
  TVB_I64 = 8,
  TVB_F64 = 9,
  TVB_BOOL = 10,
  TVB_I16 = 11,
  TVB_E4M3FNUZ = 12, /* float8_e4m3fnuz: bias 8, no infinities, no negative zero, NaN = 0x80 */
  TVB_E5M2FNUZ = 13  /* float8_e5m2fnuz: bias 16, likewise */
};

/* An allocation as seen by the host (replaces VktAlloc, vk.h:50-55: on CUDA
 * the data pointer is the device address, so `host`/`address` collapse). */
typedef struct TvbAlloc {
  void* handle;   /* pass back to tvb_free */
  void* ptr;      /* device pointer, 256-byte aligned */
  uint64_t size;  /* bytes reserved (>= requested) */
  int32_t device;
  int32_t pad;
} TvbAlloc;

/* ---- runtime (replaces vkt_last_error / vkt_alloc / vkt_free / vkt_synchronize /
 *      vkt_empty_cache / vkt_memory_stats / vkt_capabilities, vk.h:56-68) ---- */

TVB_API const char* tvb_last_error(void);
/* Number of usable sm_100 devices; -1 (with a message) if CUDA cannot start. */
TVB_API int tvb_device_count(void);
TVB_API int tvb_set_device(int device);
TVB_API int tvb_current_device(void);
TVB_API int tvb_device_name(int device, char* buf, size_t n);
/* Feature bits in the reference's layout (vk.h:97-106): always
 * float64|int16|float16|int8|bf16-matrices|shared32K = 1|2|4|8|16|32|64 on a B200. */
TVB_API uint32_t tvb_capabilities(int device);
TVB_API int tvb_alloc(int device, uint64_t nbytes, TvbAlloc* out);
/* Returns the block to the device's pool (stream-ordered). Safe after tvb_shutdown. */
TVB_API void tvb_free(void* handle);
TVB_API int tvb_synchronize(int device);
TVB_API int tvb_empty_cache(int device);
TVB_API void tvb_memory_stats(int device, uint64_t* allocated, uint64_t* reserved, uint64_t* blocks);
/* The CUDA stream (cudaStream_t) that every launcher queues on for `device`. */
TVB_API void* tvb_stream(int device);
/* Replaces the device's stream with a caller-owned one (NULL restores the runtime's own). The runtime's scratch is ordered
 * by one stream per device at a time: the new stream is made to wait for what is already queued on the old one. */
TVB_API int tvb_set_stream(int device, void* stream);
/* Kernels launched so far (the reference's dispatch_count, crates/pyvk/src/lib.rs:112-116). */
TVB_API uint64_t tvb_dispatch_count(void);
/* Waits for queued work and releases every pool and stream. */
TVB_API void tvb_shutdown(void);

/* Copies: host<->device wait for completion when the host buffer is pageable
 * (cudaMemcpyAsync semantics otherwise); device->device is stream-ordered. */
/* Capture of the device's stream into a CUDA graph (for launch-bound loops such as a decoding step): every launcher
 * called between begin and end is recorded instead of run; tvb_graph_launch replays the recording on the stream.
 * Warm every shape once before capturing (first calls allocate scratch and set kernel attributes). */
TVB_API int tvb_graph_begin(int device);
TVB_API int tvb_graph_end(int device, void** graph_exec);
TVB_API int tvb_graph_launch(int device, void* graph_exec);
TVB_API void tvb_graph_destroy(void* graph_exec);

TVB_API int tvb_memcpy_h2d(int device, void* dst, const void* src, uint64_t nbytes);
TVB_API int tvb_memcpy_d2h(int device, void* dst, const void* src, uint64_t nbytes);
TVB_API int tvb_memcpy_d2d(int device, void* dst, const void* src, uint64_t nbytes);
/* Device -> page-locked host memory without waiting: the bytes are there after tvb_synchronize (or any later
 * waiting call) on the device. */
TVB_API int tvb_memcpy_d2h_async(int device, void* dst, const void* src, uint64_t nbytes);
/* The same copy on a second stream of the runtime's (the copy-out lane): it starts when everything queued on the device's
 * stream so far has run, and what is queued afterwards does not wait for it, so a result travels to the host under the
 * next kernels. The caller leaves `src` unwritten until the lane is joined. tvb_join_copies makes the device's stream wait
 * for the lane; tvb_synchronize and tvb_graph_end join by themselves (a recorded step holds its copies). No counterpart
 * in the reference, whose stream is one queue (crates/vkcore/src/stream.rs). */
TVB_API int tvb_memcpy_d2h_overlapped(int device, void* dst, const void* src, uint64_t nbytes);
TVB_API int tvb_join_copies(int device);

/* Page-locked host memory (replaces the reference's pinned allocator, crates/pyvk/csrc/backend.cpp:313-340):
 * copies from and to it are asynchronous. tvb_host_is_pinned: 1 if `ptr` lies in page-locked memory, else 0. */
TVB_API int tvb_host_alloc(uint64_t nbytes, void** out);
TVB_API void tvb_host_free(void* ptr);
TVB_API int tvb_host_is_pinned(const void* ptr);
/* Page-locks host memory the caller owns (for instance a shared-memory segment mapped by every process of a node) and
 * returns the address under which kernels reach it. tvb_host_unregister before the memory is unmapped. */
TVB_API int tvb_host_register(void* ptr, uint64_t nbytes, void** device_ptr);
TVB_API int tvb_host_unregister(void* ptr);

/* ---- data movement kernels (the slice of the reference's cast / move / fill
 *      kernels that the four ops and their tests need: cast.slang, move.slang) */

/* dst[i...] = convert(src[i...]) over `ndim` (<= 8) dimensions with element strides. */
TVB_API int tvb_copy_strided(int device, void* dst, int dst_dtype, const int64_t* dst_strides, const void* src, int src_dtype,
                     const int64_t* src_strides, const int64_t* sizes, int ndim);
/* Every element of a strided tensor of `itemsize`-byte elements set to the low bytes of `bits`. */
TVB_API int tvb_fill_strided(int device, void* dst, int itemsize, uint64_t bits, const int64_t* strides, const int64_t* sizes,
                     int ndim);

/* c[i, j] += v[j] for a [m, n] matrix with row stride c_sm (elements): float32 addition, one rounding to c's dtype.
 * The bias of a Linear whose product has no bias operand (the reference adds it with its generic add kernel,
 * crates/pyvk/csrc/quant.cpp:296-297 does so inside _scaled_mm). float32, float16 and bfloat16, in any pairing. */
TVB_API int tvb_add_rowvec(int device, void* c, int c_dtype, int64_t c_sm, const void* v, int v_dtype, int64_t m, int64_t n);

/* ---- aten::_weight_int8pack_mm (replaces vkt_dispatch("qmm8_<f32|f16|bf16>", ...),
 *      crates/pyvk/csrc/quant.cpp:86-117; parameters as Q8Params, quant.cpp:31-37) ----
 * C[m, n] = A[m, k] @ (int8 B[n, k] * scales[n]).T, float32 accumulation, rounded once
 * to `dtype`. a_sm: A's row stride in elements (column stride 1). scales and C have A's
 * dtype; B and C are contiguous. variant: 0 automatic, 1 the plain CUDA-core kernel,
 * 2 the TMA-fed skinny kernel (m <= 64, 16-bit A, k % 128 == 0), 3 the tcgen05 kernel that widens the weights in
 * its main loop, 4 the weights widened once into runtime-owned scratch (2 bytes per weight) and the 16-bit tcgen05
 * GEMM over them (chosen from m = 1024 on), 5 float32 A on tcgen05 through an exact split of every value into three
 * bfloat16 terms (at most 256 rows, k a multiple of 64, B 16-byte aligned; chosen whenever it applies). */
TVB_API int tvb_qmm8(int device, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales, void* c,
             int64_t m, int64_t n, int64_t k, int variant);

/* ---- the same product with weights widened ahead of time (prefill: many rows of A, the same weights call after call) ----
 * tvb_qmm8_widen converts B and scales once into a caller-owned buffer of tvb_qmm8_widened_bytes(n, k) bytes (256-byte
 * aligned; n * k weights in A's 16-bit dtype, then the scales in float32); tvb_qmm8_widened multiplies with them: the
 * arithmetic of tvb_qmm8's variant 4 without its per-call pass over the weights. dtype: TVB_F16 or TVB_BF16; k % 16 == 0;
 * rows of A 16-byte aligned. (The ATen layer keeps such buffers per weight tensor, within a byte budget.) */
TVB_API uint64_t tvb_qmm8_widened_bytes(int64_t n, int64_t k);
TVB_API int tvb_qmm8_widen(int device, const int8_t* b, const void* scales, int dtype, int64_t n, int64_t k, void* widened,
                   uint64_t widened_bytes);
TVB_API int tvb_qmm8_widened(int device, const void* a, int dtype, int64_t a_sm, const void* widened, void* c, int64_t m, int64_t n,
                     int64_t k);

/* ---- the decode product with the weight rows sharded over the GPUs of one node (no counterpart in the reference,
 *      which has one device: crates/pyvk/csrc/backend.cpp:296) ----
 * Rank `rank` of `world` computes its n_local output columns and its kernel's epilogue stores them straight into
 * every rank's [m, n_local * world] output buffer at columns [rank * n_local, (rank + 1) * n_local): this GPU's own
 * memory and the peers' over NVLink (plain 16-byte stores to peer-mapped memory). c_ranks: host array of `world` device
 * pointers, entry r being rank r's output buffer as mapped into this process (tvb_ipc_export on the owner,
 * tvb_ipc_import here).
 *
 * Arrival is counted on a channel: every rank owns an array of 32 uint32 arrival counters ([4 slots][8 source ranks],
 * 16-byte aligned), zero at the start (flag_ranks: host array of `world` device pointers, entry r being rank r's array as
 * mapped here), and a uint32 product count in its own device memory, zero at the start (seq_counter). Product number q of
 * the channel (counted from zero) is reported in slot q % 4: every CTA of the product kernel, once its columns are stored
 * on every rank, adds its share to counter [q % 4][rank] of every rank's array (system scope, after a system-scope fence);
 * a product adds 1024 in all, so rank r's slice of product q has arrived here when counter [q % 4][r] of this rank's array
 * has reached 1024 * (q / 4 + 1). The kernel's last CTA adds one to the product count.
 *
 * Ordering. Before it reads A or stores a column, a product kernel waits (bounded, see tvb_set_wait_limit_ms) until all
 * ranks have delivered every earlier product of the channel; meanwhile its weights already stream into shared memory. So
 * (1) the next sharded product may take a gathered output as its A without any call in between, and (2) an output buffer
 * may be written again by the second product after the one that filled it (use two buffers in turn), provided that
 * everything else that reads it on this rank was queued before this rank's next product. `independent` = i (1 to 3)
 * relaxes the wait to all but the latest i products of the channel (a pass of 16 rows counts as a product here): for a product that neither reads the outputs of those i products nor writes a buffer that any rank
 * may still be reading while they run. Work that is not a sharded
 * product of the same channel (copies, other kernels) must be queued after tvb_wait_flags, which queues a one-warp
 * kernel that waits in the same way for all products queued so far and changes nothing. The counts live on the device,
 * so a captured CUDA graph of products can be replayed. Every rank must queue the same sequence of products on a channel.
 * A wait that runs out sets the device's status word (tvb_synchronize then fails with "status 5") and the kernels go on
 * without waiting again. 1 <= m <= 64 (16 rows of A per pass, every pass a product of its own on the channel), 16-bit A,
 * k a multiple of 128. */
TVB_API int tvb_qmm8_gather(int device, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales,
                            void* const* c_ranks, uint32_t* const* flag_ranks, int world, int rank,
                            uint32_t* seq_counter, int independent, int64_t m, int64_t n_local, int64_t k);
TVB_API int tvb_wait_flags(int device, const uint32_t* flags, int world, const uint32_t* seq_counter);

/* Several decode products of one shape in ONE launch of the decode kernel (no counterpart in the reference, which
 * dispatches once per product, crates/pyvk/csrc/quant.cpp:86-117): products that do not depend on each other, such as
 * the requests of one decoding step against different weights, or q, k, v of one layer. Product g is
 * C_g[m_g, n] = A_g[m_g, k] . B_g[n, k]^T * scales_g[n] with 1 <= m_g <= 16; n, k and the dtype (TVB_F16 / TVB_BF16)
 * are shared; k % 128 == 0, rows of A and B 16-byte aligned. The kernel numbers its tiles through all products and cuts
 * the whole list into one range per SM, so the launch costs one start and one end whatever `count` (1 to 4) is. Results
 * are those of tvb_qmm8 within one rounding of the float32 sums (the same products, summed over differently cut ranges of
 * k); a launch repeats its own results bit for bit.
 * c_ranks: tvb_qmm8_group reads c_ranks[0], the contiguous [m, n] output; it may lie in page-locked host memory
 * (tvb_host_alloc, cudaHostAlloc), in which case the kernel's stores are the copy to the host: the result is there after
 * tvb_synchronize and no tvb_memcpy_d2h is needed. tvb_qmm8_group_gather is the sharded form
 * (see tvb_qmm8_gather): n_local rows of every B on this rank, c_ranks = every rank's [m, n_local * world] buffer for that
 * product; the launch takes `count` consecutive product numbers on the channel and waits, before it reads any A, for
 * all earlier products but the latest `independent` (independent + count <= 4). */
typedef struct TvbGroupItem {
  const void* a;
  int64_t a_sm;
  const int8_t* b;
  const void* scales;
  void* const* c_ranks;
  int64_t m;
  void* c_host;  /* NULL, or one more destination for this product's columns: page-locked host memory that the device can
                  * address (tvb_host_alloc, or any host memory after tvb_host_register), laid out like the c_ranks buffers.
                  * Sharded, the ranks of a node may all pass one buffer in shared memory: every rank's kernel stores its own
                  * columns there, and after tvb_wait_flags + tvb_synchronize every process reads the whole result with no
                  * copy. Either every product of a launch has one or none. */
} TvbGroupItem;
TVB_API int tvb_qmm8_group(int device, int dtype, const TvbGroupItem* items, int count, int64_t n, int64_t k);
TVB_API int tvb_qmm8_group_gather(int device, int dtype, const TvbGroupItem* items, int count, uint32_t* const* flag_ranks, int world,
                          int rank, uint32_t* seq_counter, int independent, int64_t n_local, int64_t k);
/* How long the kernels above wait for peers before they give up (default about 2000 ms). Process-wide; applies to
 * kernels launched (or captured) afterwards. 1 <= ms <= 60000. */
TVB_API int tvb_set_wait_limit_ms(int ms);
/* ---- a list of decode products in one launch (no counterpart in the reference, which issues one dispatch per product:
 *      crates/pyvk/csrc/quant.cpp:86-117) ----
 * A chain is a fixed sequence of int8 weight-only products (the Linears of a decoder stack for one token step; the products
 * of one decoding step) that one persistent kernel walks: the weights of the next products stream into shared memory while
 * the current one is finished, so the start-up and wind-down of a launch, which cost more than a sharded decode product's
 * streaming time, are paid once per chain. Results are bit for bit those of tvb_qmm8 (m <= 16 per pass) product by product.
 *
 * tvb_qmm8_chain_create records the products: all pointers are device pointers that must stay valid (and whose contents
 * the caller may rewrite between runs); product i may take the output of product i - 1 as its A. c_ranks: host array of
 * `world` pointers to every rank's [m, n_local * world] output buffer (world == 1: one pointer, the [m, n_local] output).
 * `independent` as in tvb_qmm8_gather (0 to 3): a product starts when all earlier products of the chain, all but the latest
 * `independent`, are complete on every rank. 1 <= m <= 64 (16 rows per pass), k a multiple of 128, A's rows and B 16-byte
 * aligned; dtype TVB_F16 or TVB_BF16 for the whole chain. Sharded chains (world > 1) use the channel of tvb_qmm8_gather
 * (flag_ranks, seq_counter), on which a chain of n passes counts as n products; every rank must run the same chains in the
 * same order. With world == 1 both may be NULL (the chain then keeps counters of its own). wait_at_end != 0: the launch
 * ends only when every rank's columns of the last product have arrived in this rank's buffers, so work queued after
 * tvb_qmm8_chain_run may read them without tvb_wait_flags. tvb_qmm8_chain_run queues one cooperative launch on the device's
 * stream (capturable in a CUDA graph). All waits inside are bounded (tvb_set_wait_limit_ms); one that runs out is reported
 * by tvb_synchronize as status 5. tvb_qmm8_chain_destroy waits for the device's stream and frees the chain. */
typedef struct TvbChainItem {
  const void* a;
  int64_t a_sm;
  const int8_t* b;
  const void* scales;
  void* const* c_ranks;
  int64_t m, n_local, k;
  int32_t independent;
  int32_t reserved;
} TvbChainItem;
TVB_API int tvb_qmm8_chain_create(int device, int dtype, const TvbChainItem* items, int count, uint32_t* const* flag_ranks,
                                  int world, int rank, uint32_t* seq_counter, int wait_at_end, void** chain);
TVB_API int tvb_qmm8_chain_run(int device, void* chain);
TVB_API void tvb_qmm8_chain_destroy(void* chain);
/* ---- collectives for hosts without PyTorch (no counterpart in the reference: one device, crates/pyvk/csrc/backend.cpp:296) ----
 * The all-gather that assembles the column slices of any sharded product (tvb_qmm4*, tvb_scaled_mm, tvb_qmm8 at any m) on
 * every rank, over NCCL (looked up at run time: TVB200_NCCL_LIB, else the process's libnccl.so.2; -1 with a message where
 * there is none). One process per GPU: rank 0 makes an id (tvb_comm_unique_id, 128 bytes), the host carries it to the other
 * ranks by its own means, and every rank calls tvb_comm_init_rank. A single process that drives several GPUs calls
 * tvb_comm_init_all instead (comms_out: `ndev` handles, entry i for devices[i]). Communicators are non-blocking and every
 * call is bounded on the host: a call that gets no answer within its time limit (timeout_ms; 0: 30 s) aborts the
 * communicator and returns -1 instead of hanging, after which only tvb_comm_abort / tvb_comm_destroy may be called on it.
 * tvb_all_gather queues rank r's `nbytes` into recv[r * nbytes ...) on the device's stream; tvb_all_gather_columns does
 * the same for a [m, n_local] slice and leaves the row-major [m, n_local * world] matrix in c_full (the ranks' slices
 * interleaved by a small kernel; scratch is the runtime's). tvb_comm_wait waits for the device's stream with a limit and
 * aborts the communicator if the collective does not finish (a peer that has gone), which also lets the stream drain.
 * tvb_comm_abort frees a communicator without waiting for anybody; tvb_comm_destroy waits for queued work first. */
TVB_API int tvb_comm_unique_id(uint8_t* id128);
TVB_API int tvb_comm_init_rank(int device, const uint8_t* id128, int world, int rank, int timeout_ms, void** comm);
TVB_API int tvb_comm_init_all(const int* devices, int ndev, void** comms_out);
TVB_API int tvb_all_gather(void* comm, const void* send, void* recv, uint64_t nbytes);
TVB_API int tvb_all_gather_columns(void* comm, const void* c_local, void* c_full, int dtype, int64_t m, int64_t n_local);
TVB_API int tvb_comm_wait(void* comm, int timeout_ms);
TVB_API int tvb_comm_abort(void* comm);
TVB_API int tvb_comm_destroy(void* comm);

/* A device allocation as a 64-byte handle plus offset that another process of the node can map (cudaIpc*). */
TVB_API int tvb_ipc_export(int device, const void* ptr, uint8_t* handle64, uint64_t* offset);
TVB_API int tvb_ipc_import(int device, const uint8_t* handle64, uint64_t offset, void** out);

/* A Linear over the same product: c = round(round(round(A @ (B * scales).T) + bias[n]) + residual[m, n]), every sum rounded
 * to A's dtype as the separate steps (tvb_qmm8, tvb_add_rowvec twice) would round it, so the result is bit for bit theirs.
 * bias and residual are of A's dtype, contiguous, and either may be NULL. With at most 32 rows in a shape the decode
 * kernel takes (see tvb_qmm8) the adds happen in that kernel's epilogue, where a tile's finished sums are scaled: no
 * further launch, and c may then be the residual itself (x += proj(h) in place). Any other shape runs the product and
 * then one pass per operand. The reference has no such entry point (its op stops at the product,
 * crates/pyvk/csrc/quant.cpp:59-119); this is the caller's next step folded in. */
TVB_API int tvb_qmm8_linear(int device, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales, const void* bias,
                    const void* residual, void* c, int64_t m, int64_t n, int64_t k);

/* ---- tvb_qmm8's decode kernel for hosts that must not allocate (no counterpart in the reference) ----
 * Some hosts cannot let a library call cudaMalloc on their behalf: a serving process that handed all of HBM to its own
 * pool at start-up (so any later driver allocation fails), or one whose request path forbids calls that stall the
 * whole device while the driver maps memory. tvb_qmm8 keeps the decode kernel's partial sums and tile counters in
 * memory it allocates on first use; this entry point runs the same kernel with that scratch in an array built into the
 * library (about 5.3 MB, resident on every GPU that loads the library until the process ends) and calls no cudaMalloc,
 * cudaFree or other allocating routine. Same arguments as tvb_qmm8, with these limits, beyond which it returns -1 with
 * a message: A float16 or bfloat16, m <= 64, k a multiple of 128, A's rows and B 16-byte aligned, n <= 1 048 576, a GPU of
 * at most 160 SMs. `stream`: the cudaStream_t to queue on (NULL: the legacy default stream); the runtime's own stream is
 * not used. The first call on a device looks the array's device address up (once, with that device current) and raises
 * the kernel's shared-memory limit; make that first call before any stream capture begins. Every call uses the one
 * array: it clears the counters it needs and then relies on stream order, so two calls that can overlap on the GPU
 * (different streams, no dependency between them) race on it and must be ordered by the caller.
 * How a failure surfaces: the kernel's waits are bounded; one that runs out leaves C incomplete and sets a status word
 * inside the array (cleared at the start of every call). tvb_synchronize does not look at that word (it belongs to no
 * runtime stream); tvb_qmm8_static_scratch_status does: it waits for `stream` and stores the word of the last call on
 * `device` in *host_out (0: complete). It allocates nothing either. */
TVB_API int tvb_qmm8_static_scratch(int device, const void* a, int dtype, int64_t a_sm, const int8_t* b, const void* scales,
                                    void* c, int64_t m, int64_t n, int64_t k, void* stream);
TVB_API int tvb_qmm8_static_scratch_status(int device, void* stream, int* host_out);

/* ---- aten::_dyn_quant_pack_4bit_weight (replaces the cat of three casts,
 *      quant.cpp:139-143) ----
 * packed[0..nw) = float(weights bytes), then float(scales) [ns], then float(bias) [nbias]. */
TVB_API int tvb_qmm4_pack(int device, const uint8_t* weights, int64_t nw, const void* scales, int scales_dtype, int64_t ns,
                  const void* bias, int bias_dtype, int64_t nbias, float* packed);

/* ---- aten::_dyn_quant_matmul_4bit (replaces the two vkt_dispatch("qmm4_*") phases,
 *      quant.cpp:187-202; parameters as Q4Params, quant.cpp:39-43) ---- */

/* PHASE 0 (qmm4.slang:132-181): per-row asymmetric int8 quantisation of inp [m, k]
 * (float32 or bfloat16, contiguous). q: int8 [m, k]; recip: float [m] (1 / scale);
 * neg_zp: int32 [m] (-zero point). groupwise selects the zero point's association. */
TVB_API int tvb_qmm4_quantize(int device, const void* inp, int dtype, int64_t m, int64_t k, int groupwise, int8_t* q,
                      float* recip, int32_t* neg_zp);
/* PHASE 1 (qmm4.slang:183-247): out[m, n] from q, the rows' recip / -zp and the packed
 * float32 vector (weights' bytes as floats, scales, optional bias). iacc_out (optional,
 * int32 [m, n, k / bs]) receives every block's integer sum. */
TVB_API int tvb_qmm4_matmul(int device, const int8_t* q, const float* recip, const int32_t* neg_zp, const float* packed,
                    int has_bias, void* out, int dtype, int64_t m, int64_t n, int64_t k, int64_t bs,
                    int32_t* iacc_out);
/* Bytes of scratch tvb_qmm4 needs for an [m, k] input. */
TVB_API uint64_t tvb_qmm4_workspace_bytes(int64_t m, int64_t k);
/* Both phases; workspace: device scratch of at least tvb_qmm4_workspace_bytes(m, k). */
TVB_API int tvb_qmm4(int device, const void* inp, int dtype, const float* packed, int has_bias, void* out, int64_t m,
             int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes);

/* The same op on the tensor cores (tcgen05 kind::i8), still bit for bit: the fast route (quant.cpp:187-202 has no
 * counterpart: the reference has one kernel). `prepared` is the packed vector's weights unpacked to int8, made once
 * per packed tensor by tvb_qmm4_prepare (tvb_qmm4_prepared_bytes(n, k) bytes of device memory) and reusable for as long
 * as the packed vector does not change. Needs k and bs multiples of 32. workspace: tvb_qmm4_tc_workspace_bytes(m, k). */
TVB_API uint64_t tvb_qmm4_prepared_bytes(int64_t n, int64_t k);
TVB_API int tvb_qmm4_prepare(int device, const float* packed, int64_t n, int64_t k, int64_t bs, void* prepared,
                             uint64_t prepared_bytes);
TVB_API uint64_t tvb_qmm4_tc_workspace_bytes(int64_t m, int64_t k);
TVB_API int tvb_qmm4_tc(int device, const void* inp, int dtype, const float* packed, int has_bias, const void* prepared,
                        void* out, int64_t m, int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes);

/* The float16 form of tvb_qmm4_tc, bit for bit as well (tcgen05 kind::f16 over float16 copies of the integers: q - zero_point
 * and the weights; block sums below 2^24 are exact in the float32 accumulators). Where a block holds 32 values and every
 * scale came from bfloat16 (what the op's groupwise form is given), float(block sum) * scale is exact, so the reference's
 * multiply and add per output and block is one fma with the same single rounding: the per-block drain, which bounds both
 * forms, is a third of the int8 form's. Other scales (found when the weights are prepared) take multiply and add. `prepared`
 * comes from tvb_qmm4_prepare16 (tvb_qmm4_prepared16_bytes(n, k) bytes: two per weight). k and bs multiples of 32,
 * bs <= 8192. workspace: tvb_qmm4_tc16_workspace_bytes(m, k). */
TVB_API uint64_t tvb_qmm4_prepared16_bytes(int64_t n, int64_t k);
TVB_API int tvb_qmm4_prepare16(int device, const float* packed, int64_t n, int64_t k, int64_t bs, void* prepared,
                               uint64_t prepared_bytes);
TVB_API uint64_t tvb_qmm4_tc16_workspace_bytes(int64_t m, int64_t k);
TVB_API int tvb_qmm4_tc16(int device, const void* inp, int dtype, const float* packed, int has_bias, const void* prepared,
                          void* out, int64_t m, int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes);

/* The opt-in fast route of the same op (no counterpart in the reference): one float16 GEMM on tcgen05 over exact
 * operands, (q - zero_point) and weight * block scale, accumulated over the whole of k in float32. Outputs differ from the
 * exact routes by float32 accumulation order only (not bit for bit). tvb_qmm4_fast_prepare writes the float16 weights
 * (tvb_qmm4_fast_prepared_bytes(n, k) bytes) and, if inexact_host is not NULL, waits and stores there whether some
 * weight * scale product was not exact in float16 (then this route must not be used). k a multiple of 8. */
TVB_API uint64_t tvb_qmm4_fast_prepared_bytes(int64_t n, int64_t k);
TVB_API int tvb_qmm4_fast_prepare(int device, const float* packed, int64_t n, int64_t k, int64_t bs, void* prepared,
                                  uint64_t prepared_bytes, int* inexact_host);
TVB_API uint64_t tvb_qmm4_fast_workspace_bytes(int64_t m, int64_t k);
TVB_API int tvb_qmm4_fast(int device, const void* inp, int dtype, const float* packed, int has_bias, const void* prepared,
                          void* out, int64_t m, int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes);

/* ---- aten::_dyn_quant_matmul_4bit for at most 16 rows (decoding): the int4 weights streamed from HBM once, bit for bit
 *      the same results as tvb_qmm4 (replaces the two dispatches of crates/pyvk/csrc/quant.cpp:187-202 for small m) ----
 * tvb_qmm4_decode_usable: 1 when the kernel takes the shape (m <= 16, n % 8 == 0, k % 512 == 0, bs % 32 == 0,
 * 512 % bs == 0, and k small enough, about 8192, for its activation fragments of 16 bytes per value of k to leave room for
 * two weight records per warp in shared memory). tvb_qmm4_decode_prepare re-tiles the packed vector's weights and scales once per packed tensor
 * (0.5 byte per weight + 4 bytes per block scale; 16-byte aligned buffer of tvb_qmm4_decode_prepared_bytes). */
TVB_API int tvb_qmm4_decode_usable(int64_t m, int64_t n, int64_t k, int64_t bs);
TVB_API uint64_t tvb_qmm4_decode_prepared_bytes(int64_t n, int64_t k, int64_t bs);
TVB_API int tvb_qmm4_decode_prepare(int device, const float* packed, int64_t n, int64_t k, int64_t bs, void* prepared,
                            uint64_t prepared_bytes);
TVB_API uint64_t tvb_qmm4_decode_workspace_bytes(int64_t m, int64_t k);
TVB_API int tvb_qmm4_decode(int device, const void* inp, int dtype, const float* packed, int has_bias, const void* prepared,
                    void* out, int64_t m, int64_t n, int64_t k, int64_t bs, void* workspace, uint64_t workspace_bytes);

/* ---- aten::_scaled_mm (replaces the chain of cast / mul / matmul / add / cast
 *      dispatches, quant.cpp:283-299) ----
 * out[m, n] = cast((a * scale_a) @ (b * scale_b) + bias) (float8 outputs: times
 * 1 / *scale_result). a: float8 [m, k], element (i, kk) at a[i * a_s0 + kk * a_s1];
 * b: float8 [k, n], element (kk, j) at b[kk * b_s0 + j * b_s1] (strides in elements).
 * a_dtype / b_dtype: TVB_E4M3 or TVB_E5M2 (the tensor cores' own formats), or the fnuz formats TVB_E4M3FNUZ / TVB_E5M2FNUZ,
 * which the reference tabulates as well (crates/pyvk/csrc/backend.cpp:471-477,486-534) and which run on the plain kernel
 * (decoded in the loop; the tensor cores have no such operand format). scale_a / scale_b: device float32, one element
 * (rowwise 0) or m / n elements (rowwise 1). bias: n elements of bias_dtype, or NULL.
 * scale_result: device float32 or NULL. out: contiguous [m, n] of out_dtype (F32, F16,
 * BF16, E4M3, E5M2, E4M3FNUZ, E5M2FNUZ). variant: 0 automatic, 1 the plain kernel, 2 the tcgen05 kernels, 3 among
 * those the one that puts a pair of CTAs (tcgen05 cta_group::2) on each 256 x 256 tile, whatever the shape. */
TVB_API int tvb_scaled_mm(int device, const void* a, int a_dtype, int64_t a_s0, int64_t a_s1, const void* b, int b_dtype,
                  int64_t b_s0, int64_t b_s1, const float* scale_a, const float* scale_b, int rowwise,
                  const void* bias, int bias_dtype, const float* scale_result, void* out, int out_dtype, int64_t m,
                  int64_t n, int64_t k, int variant);

/* The same product with B's columns sharded over the GPUs of one node (no counterpart in the reference, which has one
 * device: crates/pyvk/csrc/backend.cpp:296): rank `rank` of `world` multiplies by its [k, n_local] slice of B (and its
 * n_local values of a row-wise scale_b and of the bias) and the tcgen05 kernel's epilogue stores the tile rows straight
 * into every rank's [m, n_local * world] output at columns [rank * n_local, (rank + 1) * n_local): this GPU's memory and
 * the peers' over NVLink, tile by tile while the other tiles are still being multiplied. Arrival is counted on the channel
 * of tvb_qmm8_gather (c_ranks, flag_ranks, seq_counter, independent as there; one product = one count): the kernel waits
 * for the channel's earlier products before its first store, and work that is not a sharded product of the channel must
 * be queued after tvb_wait_flags. Needs the layout of the tcgen05 kernel (K-major operands, 16-byte aligned rows). */
TVB_API int tvb_scaled_mm_gather(int device, const void* a, int a_dtype, int64_t a_s0, int64_t a_s1, const void* b, int b_dtype,
                                 int64_t b_s0, int64_t b_s1, const float* scale_a, const float* scale_b, int rowwise,
                                 const void* bias, int bias_dtype, const float* scale_result, void* const* c_ranks, int out_dtype,
                                 uint32_t* const* flag_ranks, int world, int rank, uint32_t* seq_counter, int independent,
                                 int64_t m, int64_t n_local, int64_t k);

/* ---- aten::mm / aten::addmm for float32, float16 and bfloat16 (replaces the reference's gemm dispatches,
 *      crates/pyvk/csrc/linalg.cpp:227-321, for the matrices either side of the quantised products) ----
 * out[m, n] = A[m, k] @ B[k, n] (+ bias[n]), float32 accumulation, one rounding to out_dtype. A and B have one dtype;
 * element (i, kk) of A at a[i * a_s0 + kk * a_s1], element (kk, j) of B at b[kk * b_s0 + j * b_s1]; out contiguous.
 * variant: 0 automatic, 1 the plain CUDA-core kernel (any strides, float32 included), 2 the tcgen05 kernels (16-bit
 * operands, both K-major: a_s1 == 1 and b_s0 == 1, rows 16-byte aligned), 3 among those the kernel of CTA pairs. */
TVB_API int tvb_mm(int device, const void* a, int dtype, int64_t a_s0, int64_t a_s1, const void* b, int64_t b_s0, int64_t b_s1,
           const void* bias, int bias_dtype, void* out, int out_dtype, int64_t m, int64_t n, int64_t k, int variant);

/* The same product with a matrix added before the one rounding: out = A @ B (+ bias[n]) + residual[m, n], the form
 * aten::addmm takes with a full `self` (a decoder block's residual stream added in the product's epilogue instead of by
 * a kernel of its own). Row i of the residual starts residual_ld elements after row i - 1 (>= n); its dtype is one of
 * the three floats and need not be the operands'. residual == NULL: tvb_mm. `out` may be the residual itself. */
TVB_API int tvb_addmm(int device, const void* a, int dtype, int64_t a_s0, int64_t a_s1, const void* b, int64_t b_s0, int64_t b_s1,
              const void* bias, int bias_dtype, const void* residual, int residual_dtype, int64_t residual_ld, void* out,
              int out_dtype, int64_t m, int64_t n, int64_t k, int variant);

#ifdef __cplusplus
}
#endif
#endif /* TVB200_H */
