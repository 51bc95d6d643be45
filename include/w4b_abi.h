/*
 * w4b_abi.h -- C ABI of the B200 (sm_100a) fused-dequant library, libw4b200.so.
 *
 * One entry point per host entry of the reference project's GPU API
 * (namespace w4::gpu); each declaration cites the reference interface it
 * replaces by file:line (paths relative to the reference project's root).
 * Plain pointers and sizes only; all data pointers are DEVICE pointers unless
 * a parameter is named *_host. `stream` is a cudaStream_t passed as void*
 * (NULL = the default stream). Calls are asynchronous with respect to the host
 * exactly like the reference's launchers: only launch-time errors are reported.
 *
 * Return value: W4B_OK, or
 *   W4B_INVALID  a contract violation -- what the reference reports by throwing
 *                std::invalid_argument. Detected on the host BEFORE any
 *                allocation or launch; no pointer is dereferenced.
 *   W4B_CUDA     a CUDA runtime failure -- the reference's std::runtime_error.
 * w4b_last_error() returns the message of the calling thread's last failure.
 *
 * Like the reference (include/w4/fused.cuh:51-54, include/w4/kvflash.cuh:56-57)
 * the library keeps grow-only device scratch per device; calls that use it must
 * not be in flight concurrently on different streams of one device.
 */
#ifndef W4B_ABI_H_
#define W4B_ABI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define W4B_OK 0
#define W4B_INVALID 1
#define W4B_CUDA 2

/* Which GEMM kernel serves a call. AUTO applies the library's crossover
 * (w4b_dispatch_mma_min_m); the others pin one kernel so that the reference's
 * separately addressable entries gemm_fused / gemm_mma stay addressable. */
#define W4B_PATH_AUTO 0
#define W4B_PATH_STREAM 1  /* replaces gemm_fused / gemm_fused_mx: HBM-streaming kernel   */
#define W4B_PATH_TENSOR 2  /* replaces gemm_mma / gemm_mma_mx: tcgen05 / TMEM kernel      */
#define W4B_PATH_GENERIC 3 /* shape-agnostic kernel behind both (ragged K, odd gs, ...)    */

/* Packed W4 weights. Field order and meaning of DevicePackedW
 * (include/w4/dequant.cuh:31-37); format of include/w4/pack.hpp:3-14:
 * q N*words(K) uint32, nibble j of word w is k = 8w+j, low nibble first;
 * scales N*G FP16; zeros N*words(G) uint32 (asymmetric only, NULL otherwise). */
typedef struct w4b_packed_w4 {
  int N, K, gs, G;
  int symmetric;
  const uint32_t* q;
  const uint16_t* scales; /* FP16 bit patterns */
  const uint32_t* zeros;
} w4b_packed_w4;

/* Packed MXFP4 weights: DevicePackedWm (include/w4/mxfused.cuh:26-30);
 * format of include/w4/mx.hpp:10-14: E2M1 codes packed like q above, one E8M0
 * byte per (row, 32-element block), B = ceil(K/32). */
typedef struct w4b_packed_mx {
  int N, K, B;
  const uint32_t* q;
  const uint8_t* scales;
} w4b_packed_mx;

/* W4 KV cache: DeviceKVW4 (include/w4/kvattention.cuh:39-48). H head slabs of
 * the W4 format with rows = positions and K axis = D. For the paged entry the
 * slab of one head has npages*page rows and S is the logical length. */
typedef struct w4b_kv_w4 {
  int H, S, D, gs, G;
  int symmetric;
  const uint32_t* q_k;
  const uint16_t* s_k;
  const uint32_t* z_k;
  const uint32_t* q_v;
  const uint16_t* s_v;
  const uint32_t* z_v;
} w4b_kv_w4;

/* FP8 E4M3 KV cache: DeviceKVF8 (include/w4/kvflash.cuh:390-396): one byte per
 * element [H][S][D], one FP16 scale per (position, group). */
typedef struct w4b_kv_f8 {
  int H, S, D, gs, G;
  const uint8_t* q_k;
  const uint16_t* s_k;
  const uint8_t* q_v;
  const uint16_t* s_v;
} w4b_kv_f8;

/* ---- library state ---------------------------------------------------- */

const char* w4b_last_error(void);
/* M at or above this goes to the tensor kernel under W4B_PATH_AUTO; replaces
 * the constant DISPATCH_MMA_MIN_M (include/w4/dispatch.cuh:25). */
int w4b_dispatch_mma_min_m(void);
/* Which kernel W4B_PATH_AUTO (or a pinned path) would run for this shape:
 * returns a W4B_PATH_* value >= 1, or -1 when the arguments are invalid. */
int w4b_gemm_w4_route(const w4b_packed_w4* p, int M, int path, const void* x);
int w4b_gemm_mx_route(const w4b_packed_mx* p, int M, int path, const void* x);
/* Synchronises the current device and returns the kernels' own status word:
 * 0, or a non-zero code when a bounded device-side wait gave up (the kernel
 * then returned early and its output is undefined). Clears the word. */
int w4b_device_status(void);
/* Number of kernel launches this library has issued from the calling process. */
unsigned long long w4b_launch_count(void);

/* Launch overlap between consecutive kernels of a stream (no counterpart in the reference, whose
 * launches are plainly stream-ordered). Off by default. When on, the stream GEMM is launched with
 * programmatic stream serialization: its CTAs may become resident while the previous kernel of the
 * stream is still running and pre-load the PACKED WEIGHTS (q / scales / zeros) of this call;
 * activations, outputs and library scratch are touched only after the previous kernel has completed
 * and its writes are visible. Turn it on only if no kernel writes a weight buffer directly before a
 * GEMM that reads it in the same stream (weights that are uploaded once and then only read - the
 * decode-serving case - qualify). Process-wide; returns the previous setting. */
int w4b_set_launch_overlap(int on);
int w4b_launch_overlap(void);

/* ---- fused dequant GEMM: C[M,N] = X[M,K] * dequant(W)[N,K]^T ----------- */

/* gemm / gemm_fused / gemm_mma (include/w4/dispatch.cuh:27-34,
 * include/w4/fused.cuh:172-214, include/w4/mma.cuh:234-260).
 * x: M*K FP16 row-major, c: M*N FP16 row-major. w_out (optional, N*K FP16)
 * receives every dequantised weight, bit-identical to the host dequant_all. */
int w4b_gemm_w4(const w4b_packed_w4* p, const void* x, void* c, int M, int path, void* stream,
                void* w_out);
/* gemm_mx / gemm_fused_mx / gemm_mma_mx (include/w4/dispatch.cuh:36-43,
 * include/w4/mxfused.cuh:166-198,291-307). */
int w4b_gemm_mx(const w4b_packed_mx* p, const void* x, void* c, int M, int path, void* stream,
                void* w_out);

/* The same GEMM through HOST activation / output buffers: copies x_host to the
 * device, runs w4b_gemm_w4 (weights stay resident on the device) and waits until
 * the result is in c_host. A page-locked c_host (cudaHostAlloc / cudaHostRegister)
 * is written by the kernel itself; pageable memory is filled by a copy. This is the call an application that
 * keeps activations on the host makes; the reference has no such entry (its
 * tests do the two cudaMemcpy themselves, tests/test_gpu.cu:109-113,177-181). */
int w4b_gemm_w4_hostio(const w4b_packed_w4* p, const void* x_host, void* c_host, int M, int path,
                       void* stream);

/* The stream GEMM without any allocation. It has no counterpart in the reference.
 * For callers that cannot call cudaMalloc: a process whose memory pool has claimed the
 * whole device (the allocation would fail), or a serving loop that forbids allocations
 * (and the implicit device synchronisation of cudaFree) after warm-up. The kernel's
 * scratch lives in a fixed 4.25 MiB array inside the library image, held by every device
 * that loads the library. Serves only shapes of the stream kernel (K % 512 == 0, N >= 64,
 * gs 32/64/128, 16-byte aligned q / scales / x) whose scratch fits: with passes =
 * ceil(M / 16) and mt = 2 when a pass holds more than 8 rows, passes * ceil(N/64) * 4 <=
 * 65,536 counters, passes * min(units, SMs) * mt * 4096 B <= 3 MiB of fragments and
 * passes * (K/512) * (8704 * mt + 256) B <= 1 MiB of arranged activations (e.g. M <= 16,
 * K <= 28,672, N <= 1,000,000); anything else returns W4B_INVALID. The first call on a
 * device resolves the array's address and clears its counters on the given stream: make
 * it before any stream capture. All calls share the array, which keeps the last call's
 * contents (the kernel re-zeroes the counters it used); calls that overlap on the GPU
 * race on it. */
int w4b_gemm_w4_noalloc(const w4b_packed_w4* p, const void* x, void* c, int M, void* stream);

/* ---- stand-alone dequantisation (two-pass comparator, bitwise gate) ---- */

/* dequant (include/w4/dequant.cuh:62-82): w is N*K FP16. */
int w4b_dequant_w4(const w4b_packed_w4* p, void* w, void* stream);
/* dequant_mx (include/w4/mxfused.cuh:57-69). */
int w4b_dequant_mx(const w4b_packed_mx* p, void* w, void* stream);
/* dequant_f8 (include/w4/kvflash.cuh:435-457): one head, q S*D bytes, s S*G. */
int w4b_dequant_f8(const uint8_t* q, const uint16_t* s, void* w, int S, int D, int gs, void* stream);

/* ---- device-side quantizers and KV append -------------------------------- */

/* The reference quantises on the host only; a decode loop has to quantise the new
 * token's K / V on the device. These entries run the host quantizers' arithmetic
 * (FP64, operation for operation) in CUDA kernels and produce the same bits from the
 * same values. Sources are device arrays of FP64 (`*_is_f16` == 0: what the host
 * quantizers take) or FP16 values (converted exactly). What the host quantizers throw
 * on for VALUES (NaN / infinity, a scale that overflows FP16 or underflows to zero on a
 * non-zero group, an MX exponent above 127) cannot throw here: the kernel records
 * status 501 in the device status word (w4b_device_status) and zeroes the group.
 *
 * w4b_quantize_w4: quantize (include/w4/pack.hpp:64-130); q N*words(K), scales N*G,
 *   zeros N*words(G) (asymmetric only, else NULL).
 * w4b_quantize_mx: quantize_mx (include/w4/mx.hpp:71-119); scales N*ceil(K/32) bytes.
 * w4b_quantize_f8: one side of quantize_cache_f8 (include/w4/kvfp8.hpp:70-128):
 *   rows*D bytes and rows*G FP16 scales.
 * w4b_kv_append_w4: quantises one token - k_new / v_new hold H*D values - into row
 *   `row` of every head slab of the cache p (slab_rows rows per head: S for a
 *   contiguous cache, npages*page for a paged pool, where the caller resolves
 *   row = bt[t/page]*page + t%page); the same bits quantize_cache
 *   (include/w4/kvcache.hpp:60-108) gives that position. p->S is ignored.
 * w4b_kv_append_f8: the same for an FP8 cache (contiguous: S rows per head). */
int w4b_quantize_w4(const void* w, int w_is_f16, int N, int K, int gs, int symmetric, uint32_t* q,
                    uint16_t* scales, uint32_t* zeros, void* stream);
int w4b_quantize_mx(const void* w, int w_is_f16, int N, int K, uint32_t* q, uint8_t* scales, void* stream);
int w4b_quantize_f8(const void* x, int x_is_f16, int rows, int D, int gs, uint8_t* q, uint16_t* scales,
                    void* stream);
int w4b_kv_append_w4(const w4b_kv_w4* p, long long row, long long slab_rows, const void* k_new,
                     const void* v_new, int new_is_f16, void* stream);
int w4b_kv_append_f8(const w4b_kv_f8* p, long long row, const void* k_new, const void* v_new,
                     int new_is_f16, void* stream);

/* ---- offline re-layout of packed weights -------------------------------- */

/* No counterpart in the reference (its kernels take any K with scalar loads;
 * include/w4/fused.cuh:175-193 only asks for K >= 1). The fast kernels here are
 * fed by TMA and need 16-byte row pitches and K % 512 == 0 (tensor kernel:
 * K % 32 == 0); any other K runs the shape-agnostic kernels, far below the
 * memory rate. These entries convert such a matrix once: the destination is the
 * SAME matrix in the SAME packed format with K extended to dst->K by columns
 * that dequantise to +0 exactly (the zero point, 8, or E2M1 +0 inside the
 * source's partial last group; scale 0 / 2^0 with zero codes in new groups),
 * so every entry of this library accepts it like any other descriptor.
 *
 * w4b_relayout_k: the K to convert to - the next multiple of 512 (-1: K < 1).
 * w4b_relayout_w4 / _mx: src and dst are full descriptors; the caller owns the
 *   destination buffers (q N*words(dst->K), scales N*dst->G, zeros N*words(dst->G);
 *   MX: scales N*dst->B bytes) and fills N, gs, mode as in src, K = the extended
 *   K, G / B consistent with it. Every destination word is written. dst->K may
 *   be any value >= src->K. In place is rejected.
 * w4b_gemm_w4_padded / _mx_padded: gemm / gemm_mx for activations of K_x <= p->K
 *   columns (x: M rows of K_x FP16 values, the original K): a kernel copies them
 *   into library scratch with zeros behind column K_x, then the GEMM of p runs.
 *   The weight columns K_x.. meet zeros only, so the result is the product with
 *   the original matrix. A caller that keeps its activations in rows of p->K
 *   values, zeros behind K_x, calls w4b_gemm_w4 directly and saves that kernel.
 *   No w_out hook here. */
int w4b_relayout_k(int K);
int w4b_relayout_w4(const w4b_packed_w4* src, const w4b_packed_w4* dst, void* stream);
int w4b_relayout_mx(const w4b_packed_mx* src, const w4b_packed_mx* dst, void* stream);
int w4b_gemm_w4_padded(const w4b_packed_w4* p, const void* x, int K_x, void* c, int M, int path, void* stream);
int w4b_gemm_mx_padded(const w4b_packed_mx* p, const void* x, int K_x, void* c, int M, int path, void* stream);

/* ---- decode attention, one query token per head ----------------------- */

/* attention_fp16_flash (include/w4/kvflash.cuh:365-384): q H*D, k16/v16
 * [H][S][D] FP16, out H*D FP16. */
int w4b_attn_flash_fp16(const void* q, const void* k16, const void* v16, void* out, int H, int S,
                        int D, void* stream);
/* attention_w4_flash (include/w4/kvflash.cuh:350-363). k_out / v_out (optional,
 * H*S*D FP16 each) receive the dequantised cache, bit-identical to dequant_head. */
int w4b_attn_flash_w4(const w4b_kv_w4* p, const void* q, void* out, void* stream, void* k_out,
                      void* v_out);
/* attention_f8_flash (include/w4/kvflash.cuh:572-590). */
int w4b_attn_flash_f8(const w4b_kv_f8* p, const void* q, void* out, void* stream, void* k_out,
                      void* v_out);
/* attention_w4_flash_paged (include/w4/kvflash.cuh:725-764): logical position t
 * of every head lives at pool row bt[t/page]*page + t%page; bt has
 * ceil(S/page) int32 entries on the device; hooks write in logical order. */
int w4b_attn_flash_w4_paged(const w4b_kv_w4* p, const int* bt, int page, int npages, const void* q,
                            void* out, void* stream, void* k_out, void* v_out);
/* Batched form of the paged entry; it has no counterpart in the reference, whose
 * attention_w4_flash_paged (include/w4/kvflash.cuh:725-764) takes one sequence (one
 * block table) per call. nseq sequences share one pool: sequence i has seq_lens[i]
 * positions (device array, 1 <= seq_lens[i] <= max_seq_len; max_seq_len is a host
 * value that sizes the launch) and the block table bt + i * bt_stride (device,
 * bt_stride >= ceil(max_seq_len / page)); q and out are [nseq][H][D]. One slice pass
 * and one combine serve all sequences. For pages that are a power of two >= 16, eight
 * consecutive sequences of equal length ride one CTA, and a 16-position block whose
 * page is the same in all their tables (a shared prefix) is loaded and decoded once
 * for the eight - nothing has to be declared, the tables are compared. out[i] is the
 * same computation as w4b_attn_flash_w4_paged on sequence i (same kernels, same
 * rel L2 <= 1e-3 against the FP64 reference) with the sequence cut into slices for
 * ceil(nseq / 8) * H rows instead of H, so the bits agree when nseq == 1; they depend
 * on nseq and the sequence's own length only, never on the other sequences of the
 * call. p->S is ignored. Served for D = 64 / 128,
 * gs = 32 / 64 / 128 and 16-byte aligned caches and q; other shapes return
 * W4B_INVALID (call the per-sequence entry). seq_lens and bt contents are not
 * validated. */
int w4b_attn_flash_w4_paged_batched(const w4b_kv_w4* p, const int* bt, int bt_stride, const int* seq_lens,
                                    int nseq, int max_seq_len, int page, int npages, const void* q,
                                    void* out, void* stream);
/* attention_fp16 / attention_w4 (include/w4/kvattention.cuh:226-248): the
 * legacy single-block entries; same results contract, and they keep the
 * reference's S <= 4096 and D <= 512 rejections. */
int w4b_attn_single_fp16(const void* q, const void* k16, const void* v16, void* out, int H, int S,
                         int D, void* stream);
int w4b_attn_single_w4(const w4b_kv_w4* p, const void* q, void* out, void* stream, void* k_out,
                       void* v_out);

/* ---- all-gather of the sharded GEMM's output over NVLink peer memory ----- */

/* These eight entries have no counterpart in the reference (it is single-GPU). They
 * are the exchange step of the column-parallel GEMM: one process per GPU, every
 * rank owns an arena that its peers map through CUDA IPC, and one launch per step
 * stores this rank's output slice into every peer's arena with plain peer stores
 * and posts a step flag. Before storing, a step waits (bounded, ~1 s, then the
 * device status word is set) for the peers' slices of the step before the previous
 * one, so ranks stay within two steps of each other; with wait_now != 0 it also waits for the
 * peers' slices of its own step (a complete all-gather in one launch).
 * w4b_allgather_wait does that wait on its own: after it, every slice of the last
 * pushed step is in this rank's arena. Graph-capturable: step numbers come from a
 * counter in the arena. world <= 8. With wait_now == 0 the caller rotates over
 * three slice buffers (a slice is then never overwritten while a peer may read
 * it); with wait_now != 0 two suffice.
 *
 * w4b_peer_alloc: cudaMalloc + zero-fill an arena and return its 64-byte IPC handle.
 * w4b_peer_open / _close: map / unmap a peer's arena from its handle.
 * w4b_allgather_push: dst[p] = where the slice goes in rank p's arena, flag_dst[p] =
 *   rank p's 64-bit flag word for this rank (entries [rank] are ignored),
 *   flags_local = this rank's flag words (world x uint64), counters = world zero-
 *   initialised uint64 in this rank's arena. dst, flag_dst are HOST arrays of device
 *   pointers. */
int w4b_peer_alloc(size_t bytes, void** ptr, void* handle64);
int w4b_peer_open(const void* handle64, void** ptr);
int w4b_peer_close(void* ptr);
int w4b_peer_free(void* ptr);
int w4b_allgather_push(const void* src, size_t bytes, void* const* dst, void* const* flag_dst,
                       const void* flags_local, void* counters, int rank, int world, int wait_now,
                       void* stream);
int w4b_allgather_wait(const void* flags_local, const void* counters, int rank, int world, void* stream);
/* The sharded GEMM and its exchange in ONE kernel (no reference counterpart): w4b_gemm_w4 through the
 * stream kernel (M <= 16, a shape that kernel serves) into c (this rank's slice buffer in its own arena,
 * 16-byte aligned); the warp that finishes the grid's last tile then copies the slice to c_peer[p], the
 * same buffer in rank p's arena, with plain 16-byte peer stores and posts the step to flag_dst[p] exactly as
 * w4b_allgather_push does (same flags, same counters: the two entries can be mixed, and
 * w4b_allgather_wait completes a sequence). Before the first peer store the kernel waits (bounded) for the
 * peers' slices of the previous step, so ranks stay within one step of each other; rotate over three slice
 * buffers. done: a zero-initialised 32-bit word in this rank's arena. c_peer, flag_dst are HOST arrays of
 * device pointers (entries [rank] ignored). */
/* The sharded GEMM of step i with the exchange of step i - 1 inside it (no reference counterpart): w4b_gemm_w4
 * through the stream kernel (M <= 16) into c, while one otherwise idle warp per CTA copies its share of
 * `prev` - this rank's finished slice of the previous step, prev_bytes bytes in its own arena - to
 * prev_peer[p], the same buffer in rank p's arena, and the last of them posts that step to flag_dst[p] (same
 * flags and counters as w4b_allgather_push, with which it can be mixed; flow control as there). The
 * transfer rides under the streaming of this step's weights: no separate launch, no end-of-kernel fence.
 * prev_bytes == 0 carries nothing (the first step); the last step's slice is delivered by
 * w4b_allgather_push, and w4b_allgather_wait completes a sequence. Rotate over three slice buffers. */
int w4b_gemm_w4_carry(const w4b_packed_w4* p, const void* x, void* c, int M, const void* prev, size_t prev_bytes,
                      void* const* prev_peer, void* const* flag_dst, const void* flags_local, void* counters,
                      void* done, int rank, int world, void* stream);
int w4b_gemm_w4_push(const w4b_packed_w4* p, const void* x, void* c, int M, void* const* c_peer,
                     void* const* flag_dst, const void* flags_local, void* counters, void* done, int rank,
                     int world, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* W4B_ABI_H_ */