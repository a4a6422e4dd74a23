/*
 * feather_b200 -- C ABI of the packed-FP8 matrix-vector path for NVIDIA B200
 * (sm_100a).  One shared library, plain pointers and sizes, no C++ types.
 *
 * The reference project (SuriyaaMM/feather) is pure Python and has no FFI
 * layer; each entry point below names the reference function whose work it
 * replaces (paths inside the reference project).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller.  The library
 *     never allocates or frees device memory and keeps no per-call state.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default
 *     stream).  All work is enqueued on it; no call synchronises the host.
 *   - A "word" is a little-endian uint32 holding four FP8 codes, element 4k in
 *     the low byte (feather/packers/fp8.py:123-134).
 *   - mode:   0 = E5M2, 1 = E4M3 (the "fn" flavour: no inf, 0x7F/0xFF NaN).
 *   - Return: FEATHER_OK (0) or a negative feather_status; see
 *     feather_strerror().  No exceptions, no prints, no exit().
 */
#ifndef FEATHER_B200_H
#define FEATHER_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum feather_status {
    FEATHER_OK = 0,
    FEATHER_ERR_BAD_ARG = -1,     /* null pointer, negative size, N % 4 != 0 ... */
    FEATHER_ERR_MISALIGNED = -2,  /* pointer not aligned as documented          */
    FEATHER_ERR_MODE = -3,        /* unknown mode / dtype / semantics value     */
    FEATHER_ERR_ARCH = -4,        /* current device is not compute capability 10.x */
    FEATHER_ERR_LAUNCH = -5,      /* CUDA reported a launch error               */
    FEATHER_ERR_WORKSPACE = -6,   /* workspace missing or too small             */
    FEATHER_ERR_TIMEOUT = -7,     /* a bounded device-side wait gave up         */
    FEATHER_ERR_BOUNDS = -9,      /* -DFEATHER_DEBUG_BOUNDS build: an index left its buffer */
    FEATHER_ERR_TOO_LARGE = -8    /* beyond what the entry point covers: built-in scratch, inbox, resident grid, model dimension */
} feather_status;

#define FEATHER_MODE_E5M2 0
#define FEATHER_MODE_E4M3 1
#define FEATHER_SRC_F16 0
#define FEATHER_SRC_F32 1
#define FEATHER_DECODE_KERNEL 0 /* values the GEMV/dot kernels multiply with  */
#define FEATHER_DECODE_IEEE 1   /* values the reference CPU unpacker returns   */

/* Library version: major * 10000 + minor * 100 + patch. */
int feather_version(void);

/* 1 if the library was built with -DFEATHER_DEBUG_BOUNDS (every global-memory
 * index of the GEMV kernels checked on the device, violations reported by
 * feather_device_status() as FEATHER_ERR_BOUNDS), else 0.  No counterpart in
 * the reference. */
int feather_debug_bounds(void);

/* Static, NUL-terminated description of a feather_status value. */
const char* feather_strerror(int status);

/*
 * Encode fp16/fp32 values to FP8 and pack four codes per word.
 * Replaces feather/packers/fp8.py:260-281 (pack_fp8_tensor), :178-210
 * (pack_fp8_ndarray: flatten, zero-pad the tail to a whole word) and :69-136
 * (pack_fp8_into_fp32: one round-to-nearest-even cast, E4M3 overflow to the
 * NaN code, E5M2 overflow to inf).  Bit-exact with the reference packer.
 *   src      n_elems values of src_dtype (FEATHER_SRC_F16 / _F32), element
 *            aligned
 *   dst      ceil(n_elems / 4) words, 4-byte aligned; padding codes are 0
 */
int feather_encode_fp8(const void* src, int src_dtype, uint32_t* dst, int64_t n_elems,
                       int mode, void* stream);

/*
 * Decode packed words to fp32, element order.
 * FEATHER_DECODE_KERNEL reproduces the in-kernel decode of
 * feather/routines/gemv.py:31-34 (E5M2: fp16 bits = code << 8) and
 * gemv.py:83-88 (E4M3 re-bias: exponent-0 codes give +-m * 2^-17, 0x7F/0xFF
 * give +-480).  FEATHER_DECODE_IEEE reproduces the CPU unpacker
 * feather/packers/fp8.py:336-392 / :395-432.
 *   src      ceil(n_elems / 4) words;  dst  n_elems floats
 */
int feather_decode_fp8(const uint32_t* src, float* dst, int64_t n_elems, int mode,
                       int semantics, void* stream);

/*
 * Single-head, non-causal attention on packed E5M2 operands:
 *   out = softmax(Q K^T / sqrt(d)) V,  d = 4 * h_dim_words
 * Replaces _flash_attention_fp8_e5m2_acc_fp32_kernel and
 * flash_attention_fp8_e5m2_acc_fp32_gpu(q, k, v, seq_len, h_dim)
 * (feather/routines/attention.py:14-108, :110-179) with the same arithmetic:
 * key tiles of 64, FP32 scores and softmax state, probabilities rounded to FP16
 * before they multiply V.  Like the reference, keys past seq_len in the last
 * tile of 64 are read as zeros and NOT masked: each enters the softmax with
 * score 0 and value 0, so a seq_len that is not a multiple of 64 does not give
 * the textbook result (the reference's README lists the routine as unfinished).
 *   q, k, v      seq_len rows of h_dim_words packed words each
 *   out          seq_len x (4 * h_dim_words) floats, 16-byte aligned
 *   h_dim_words  a power of two from 4 to 128 (d = 16 .. 512, which covers the
 *                reference's benchmark shapes 64, 256 and 512); larger powers
 *                of two return FEATHER_ERR_TOO_LARGE, anything else
 *                FEATHER_ERR_BAD_ARG
 */
int feather_attention_fp8_e5m2(const uint32_t* q, const uint32_t* k, const uint32_t* v, float* out,
                               int64_t seq_len, int64_t h_dim_words, void* stream);

/*
 * ReLU on unpack: dst[i] = max(0, decode(code i)) as FP32, for i < n_elems.
 * Replaces _relu_1d_fp8_ret_fp32_kernel / relu1d_fp8_ret_fp32_feather_gpu
 * (feather/routines/activations.py:8-29, :32-41), which exist for E5M2 only;
 * E4M3 uses the GEMV kernels' decode (feather/routines/gemv.py:83-88) and is an
 * extension.  max has the compiled kernel's semantics: a NaN code gives 0
 * (the other operand), -0 gives +0.
 *   src  ceil(n_elems / 4) packed words, 4-byte aligned
 *   dst  n_elems floats (the reference always writes 4 per word; here the
 *        last word may be cut short)
 */
int feather_relu_fp8(const uint32_t* src, float* dst, int64_t n_elems, int mode, void* stream);

/*
 * out[r] = sum_j decode(m[r, j]) * decode(v[j]),  FP32 products and sums.
 * Replaces feather/routines/gemv.py:136-184 (gemv_fp8_e5m2_acc_fp32_gpu) and
 * :187-235 (gemv_fp8_e4m3_acc_fp32_gpu) with their kernels gemv.py:8-61 and
 * :91-133.
 *   m        M * N / 4 words, row-major, row stride N / 4 words (gemv.py:18)
 *   v        N / 4 words
 *   out      M floats (written, not accumulated)
 *   M, N     UNPACKED matrix shape; N % 4 == 0 (rows are whole words,
 *            gemv.py:182).  M == 0 or N == 0 is allowed (N == 0 writes zeros).
 * m, v and out must be 4-byte aligned; the fast paths need m 16-byte aligned
 * and N % 16 == 0, other shapes take a slower general kernel.
 * The kernel is launched with programmatic stream serialisation: it orders
 * itself after all earlier work of the stream before touching memory, and
 * lets the next kernel of the stream start its launch early.
 * The sum order differs from the reference's (which is itself unspecified);
 * results agree to FP32 rounding.
 */
int feather_gemv_fp8(const uint32_t* m, const uint32_t* v, float* out, int64_t M, int64_t N,
                     int mode, void* stream);

/*
 * feather_gemv_fp8 with option flags.
 *   FEATHER_GEMV_STATIC_MATRIX  the caller promises that no earlier work of the
 *       stream that may still be running WRITES THE MATRIX (weights that were
 *       packed once and synchronised, the usual case for repeated GEMVs).
 *       The kernel then begins streaming matrix bytes as soon as it is
 *       scheduled, before it has waited for the previous kernel of the stream;
 *       the vector is still read, and the output written, only after that
 *       wait.  Back-to-back GEMVs overlap one kernel's tail with the next
 *       one's start.  If the promise is broken (for example the matrix is
 *       packed by the kernel right before), the result is undefined; use flags
 *       = 0 there.  The reference has no counterpart (one Triton launch per
 *       call, gemv.py:181).
 */
#define FEATHER_GEMV_STATIC_MATRIX 1u
int feather_gemv_fp8_ex(const uint32_t* m, const uint32_t* v, float* out, int64_t M, int64_t N,
                        int mode, uint32_t flags, void* stream);

/*
 * GEMV against B vectors in one pass over the matrix:
 *   out[b * M + r] = sum_j decode(m[r, j]) * decode(v[b * N/4 words + j])
 * The reference multiplies one vector per launch (feather/routines/gemv.py:136,
 * :187), so B right-hand sides read the matrix B times; here each 16-byte chunk
 * of a row is loaded and decoded once for up to four vectors (B > 4 runs
 * ceil(B / 4) passes).  Per vector the result is what feather_gemv_fp8 gives
 * (the same bits where that call takes the warp-owned-rows kernel, otherwise
 * the same sums in another order).
 *   v    B packed vectors of N / 4 words, one after the other
 *   out  B rows of M floats
 *   B    0 .. 64; rows that are not whole 16-byte chunks (N % 16 != 0 or m not
 *        16-byte aligned) fall back to one single-vector GEMV per vector
 *   flags as feather_gemv_fp8_ex
 */
int feather_gemv_fp8_multi(const uint32_t* m, const uint32_t* v, float* out, int64_t M, int64_t N,
                           int B, int mode, uint32_t flags, void* stream);

/*
 * The GEMV with its result re-encoded to packed FP8: out_words receives
 * ceil(M / 4) words holding encode(out[0..M)) in `out_mode`, the tail padded
 * with zero codes -- exactly feather_encode_fp8 applied to feather_gemv_fp8's
 * FP32 result, i.e. the packed activation the next GEMV of a chain takes.  No
 * reference counterpart: there the FP32 result goes back through the CPU
 * packer (feather/packers/fp8.py:260-281) before it can feed
 * feather/routines/gemv.py:136 again.
 *   workspace   M floats, or NULL.  Matrices of N % 16 == 0 with 16-byte aligned
 *               rows that do not take the large-matrix kernel encode in the
 *               GEMV kernel's epilogue and ignore it
 *               (feather_gemv_fp8_packed_workspace_bytes returns 0 for their
 *               (M, N)); all others write their sums there and the encoder
 *               runs behind the GEMV on the same stream.  FEATHER_ERR_WORKSPACE
 *               if it is needed and NULL.
 *   flags       as feather_gemv_fp8_ex
 */
int feather_gemv_fp8_packed(const uint32_t* m, const uint32_t* v, uint32_t* out_words,
                            void* workspace, int64_t M, int64_t N, int mode, int out_mode,
                            uint32_t flags, void* stream);
int64_t feather_gemv_fp8_packed_workspace_bytes(int64_t M, int64_t N);

/*
 * One rank of a row-sharded GEMV with the gather of the output slices fused
 * into the kernel.  The reference is single-GPU (feather/routines/gemv.py:136,
 * :187 hard-code one device); rows are independent, so rank r of `world` holds
 * the packed rows [r * rows_local, (r + 1) * rows_local) and the whole packed
 * vector.  Instead of a separate all-gather, every finished row is stored into
 * ALL ranks' output buffers through peer-mapped pointers (NVLink), the rank
 * then publishes `epoch` in every rank's flag block and waits, for at most two
 * seconds, until every rank has published the same epoch in its own block.
 * When the kernel ends, peer_out[rank] holds all world * rows_local results.
 *   m_local     rows_local * N / 4 words, 16-byte aligned; N % 16 == 0,
 *               N >= 4096, rows_local >= 32 * SM count (use
 *               feather_gemv_fp8_sharded_supported(); other shapes return
 *               FEATHER_ERR_BAD_ARG: run feather_gemv_fp8 and gather instead)
 *   peer_out    HOST array of `world` device pointers: rank p's output buffer
 *               (world * rows_local floats), as mapped into THIS process
 *   peer_flags  HOST array of `world` device pointers: rank p's flag block,
 *               32 words, zero before the first call
 *   epoch       1 for the first call, +1 for every later call, equal on all
 *               ranks.  Use two output buffers alternately (even / odd epoch):
 *               a fast rank may start writing call k+1 while a slow rank's
 *               consumer still reads call k.  A rank stores call k+2 into the
 *               peers' buffers only once every peer has delivered call k+1,
 *               i.e. has been launched for it: the result of call k is valid
 *               until THIS rank's call k+1 is enqueued, not longer.  Because
 *               the epoch is a launch
 *               argument, a captured CUDA graph of this call must not be
 *               replayed (the second replay would find its epoch already
 *               published and not wait); launch it from the stream.
 * One call per rank must be in flight at the same time on every rank, each on
 * its own GPU.  A rank that never arrives makes the others raise the status
 * word after the bounded wait (see feather_device_status) instead of hanging.
 */
int feather_gemv_fp8_sharded(const uint32_t* m_local, const uint32_t* v, int64_t rows_local,
                             int64_t N, int mode, float* const* peer_out,
                             uint32_t* const* peer_flags, int rank, int world, uint32_t epoch,
                             void* stream);
int feather_gemv_fp8_sharded_supported(int64_t rows_local, int64_t N);

/*
 * feather_gemv_fp8_sharded with options.  No reference counterpart, as above.
 *   flags   FEATHER_GEMV_STATIC_MATRIX  as feather_gemv_fp8_ex.
 *           FEATHER_SHARDED_NO_WAIT     split-phase completion: the kernel ends
 *             once this rank's rows and its epoch are on their way to the
 *             peers; it does NOT wait for the peers' slices.  The caller runs
 *             feather_gemv_fp8_sharded_wait(..., epoch, ...) on the same stream
 *             before anything reads the result.  Exchange latency and the skew
 *             between ranks then overlap the next call (or whatever else the
 *             stream holds) instead of ending every call.  Results stay valid
 *             until this rank's next sharded call is enqueued, as above.
 *   stamps  NULL, or 3 device uint64 (8-byte aligned) that receive the GPU's
 *           nanosecond timer from the rank's last CTA: [0] all rows pushed,
 *           [1] epoch published, [2] all ranks' epochs seen (written by the
 *           kernel without NO_WAIT, else by feather_gemv_fp8_sharded_wait).
 *           For measuring how a step's time splits into fence / flag latency
 *           and waiting for the slowest rank.
 * feather_gemv_fp8_sharded_wait enqueues a one-warp kernel that returns when
 * every rank's epoch in peer_flags[rank] has reached `epoch` (bounded like the
 * other waits; see feather_device_status).
 */
#define FEATHER_SHARDED_NO_WAIT 2u
int feather_gemv_fp8_sharded_ex(const uint32_t* m_local, const uint32_t* v, int64_t rows_local,
                                int64_t N, int mode, float* const* peer_out,
                                uint32_t* const* peer_flags, int rank, int world, uint32_t epoch,
                                uint32_t flags, uint64_t* stamps, void* stream);
int feather_gemv_fp8_sharded_wait(uint32_t* const* peer_flags, int rank, int world, uint32_t epoch,
                                  uint64_t* stamps, void* stream);

/*
 * One rank of a COLUMN-sharded GEMV with the all-reduce of the partial results
 * fused into the kernel.  No reference counterpart (the reference is
 * single-GPU, feather/routines/gemv.py:136, :187); it is the split a
 * tensor-parallel layer needs when the vector arrives sharded: rank r holds
 * columns [r * N_local, (r + 1) * N_local) of all M rows, packed row-major with
 * row stride N_local / 4 words, and the matching N_local / 4 words of the
 * vector.  Each rank's row sums are partial.  Every CTA of the kernel stores
 * its rows' sums into all peers' inboxes through peer-mapped pointers, as
 * 8-byte (sum, call number) pairs, polls its own inbox until the peers' pairs
 * for those rows carry this call's number (bounded, see
 * feather_set_wait_limit_ms) and adds them in rank order:
 * result[i] = ((p0[i] + p1[i]) + p2[i]) + ..., the same bits on every rank.
 *   m_local     M * N_local / 4 words, 16-byte aligned; N_local % 16 == 0
 *   v_local     N_local / 4 words
 *   result      M floats, local
 *   peer_inbox  HOST array of `world` device pointers: rank p's inbox of
 *               `inbox_floats` floats, 16-byte aligned, zero before the first
 *               call, as mapped into THIS process.  Two halves are used by
 *               alternate calls; a half holds one slot per rank of
 *               2 * roundup(M, 16) floats.  inbox_floats / 2 smaller than
 *               world slots returns FEATHER_ERR_TOO_LARGE, and so does an M
 *               whose CTAs (8 or 16 rows each) do not fit the GPU at once: the
 *               CTAs wait for one another across ranks.
 *   peer_flags  HOST array of `world` device pointers: rank p's flag block, 32
 *               words, zero before the first call (only the rank's own block
 *               is used: the call counter lives there, so there is no epoch
 *               argument and a captured CUDA graph of calls can be replayed).
 *               Every rank must issue the same sequence of calls on a given
 *               inbox / flag block; M may differ from call to call,
 *               inbox_floats may not.
 * One call per rank must be in flight at the same time on every rank, each on
 * its own GPU.  A rank that never arrives makes the others raise the status
 * word after the bounded wait (see feather_device_status) instead of hanging.
 */
int feather_gemv_fp8_allreduce(const uint32_t* m_local, const uint32_t* v_local, float* result,
                               int64_t M, int64_t N_local, int mode, float* const* peer_inbox,
                               int64_t inbox_floats, uint32_t* const* peer_flags, int rank,
                               int world, void* stream);

/*
 * Let kernels on the CURRENT device load and store memory that lives on
 * `peer_device` (cudaDeviceEnablePeerAccess; already-enabled is success).  The
 * fused sharded GEMV stores into its peers' buffers, so each rank calls this
 * once per peer before its first feather_gemv_fp8_sharded.  Mapping a peer's
 * buffer into the process (CUDA IPC) does not by itself grant that access.
 * FEATHER_ERR_BAD_ARG if the two GPUs have no direct path.
 */
int feather_enable_peer_access(int peer_device);

/*
 * Sharing a buffer between the one-process-per-GPU ranks of a node (CUDA IPC),
 * for the peer_out / peer_flags arguments above.  The library allocates
 * nothing: the owner exports a buffer it already holds, the peers map it.
 *   feather_ipc_export  owner side, owner's device current.  `ptr` lies in a
 *                       cudaMalloc allocation (a PyTorch tensor of the default
 *                       allocator does); writes the 64-byte handle of that
 *                       allocation and ptr's offset inside it.
 *   feather_ipc_open    peer side, with the device that will RUN THE KERNEL
 *                       current: maps the allocation for that device (peer
 *                       access is enabled by the runtime) and returns the
 *                       address that corresponds to the owner's `ptr`.
 *   feather_ipc_close   unmaps; pass what feather_ipc_open returned and the
 *                       same offset.  The owner must keep the buffer alive
 *                       until every peer has closed it.
 */
int feather_ipc_export(const void* ptr, void* handle64, int64_t* offset);
int feather_ipc_open(const void* handle64, int64_t offset, void** mapped);
int feather_ipc_close(void* mapped, int64_t offset);

/*
 * Health check for the kernels that wait on shared-memory barriers (the large
 * GEMV streams the matrix through a ring of asynchronous bulk copies).  Every
 * such wait is bounded; a wait that gives up raises a sticky status word on
 * the device instead of hanging.  This call SYNCHRONISES `stream`, returns
 * FEATHER_ERR_TIMEOUT if the word was raised since the last check (and clears
 * it), FEATHER_OK otherwise.  No counterpart in the reference (its Triton
 * kernels have no waits); the GEMV results of a run that reports a timeout
 * are undefined.
 */
int feather_device_status(void* stream);

/*
 * Change, on the current device, how long a bounded device-side wait may go
 * without progress before it gives up (default 2000 ms; 1 .. 600000).  Takes
 * effect for kernels launched afterwards; synchronises the device.
 */
int feather_set_wait_limit_ms(int milliseconds);

/*
 * A table of GEMVs in ONE persistent launch (batch-1 decoding: one token of a
 * model is a chain of small GEMVs that, launched one by one, are bound by
 * launch and pipeline-fill latency instead of HBM).  No counterpart in the
 * reference, where every GEMV is its own launch of feather/routines/gemv.py:136
 * / :187; every op computes what feather_gemv_fp8 (or, with out_mode >= 0,
 * feather_gemv_fp8_packed) computes for the same operands, bit for bit.
 *
 * feather_chain_op describes one GEMV:
 *   m, v, out  as for feather_gemv_fp8; m and v 16-byte aligned; out holds M
 *              floats (out_mode = -1) or ceil(M / 4) packed words of the sums
 *              encoded to out_mode (FEATHER_MODE_E5M2 / _E4M3), padding codes 0
 *   M, N       N a multiple of 16, at most 8192 (FEATHER_ERR_TOO_LARGE beyond)
 *   mode       decode of m and v
 *   wait_op    -1, or the index of an EARLIER op of the table whose output is
 *              this op's vector: v is read only after that op has finished on
 *              every SM.  Ops without it may run in any overlap; an op must
 *              not read what another op of the same launch writes unless it
 *              names that op here.
 *
 * feather_gemv_chain_plan validates a HOST array of ops and writes the device
 * table (and the zeroed completion counters) into `plan`, a device buffer of
 * at least feather_gemv_chain_plan_bytes(n_ops) bytes, 16-byte aligned, owned
 * by the caller; it synchronises `stream`, so the host array may be freed on
 * return.  feather_gemv_chain_fp8 enqueues the launch; the same plan can be
 * launched again and again (also from a captured CUDA graph), but not by two
 * launches that overlap on the GPU.  FEATHER_GEMV_STATIC_MATRIX promises that
 * no work in flight writes the matrices or the plan.  Device-side waits are
 * bounded (feather_set_wait_limit_ms, feather_device_status).
 */
typedef struct feather_chain_op {
    const uint32_t* m;
    const uint32_t* v;
    void* out;
    int32_t M, N;
    int32_t mode;
    int32_t out_mode;
    int32_t wait_op;
    int32_t allreduce;  /* 0, or 1 for a column-sharded op of a tensor-parallel launch (below) */
} feather_chain_op;

int64_t feather_gemv_chain_plan_bytes(int32_t n_ops);
int feather_gemv_chain_plan(const feather_chain_op* ops, int32_t n_ops, void* plan, int64_t plan_bytes,
                            void* stream);
int feather_gemv_chain_fp8(const void* plan, int32_t n_ops, uint32_t flags, void* stream);

/*
 * The chain as one rank of a tensor-parallel group, one launch per GPU and
 * token.  No counterpart in the reference (single-GPU).  Ops with allreduce = 0
 * are local (e.g. this rank's ROWS of a projection).  An op with allreduce = 1
 * is COLUMN-sharded as in feather_gemv_fp8_allreduce: m holds this rank's
 * column block of all M rows (row stride N / 4 words, N the LOCAL column
 * count), v the matching slice of the vector; the row sums are partial and the
 * op's output is their sum over the ranks, added in rank order -- the same
 * bits on every rank.  The exchange runs inside the kernel through peer-mapped
 * inboxes ((sum, call number) pairs; no collective launch, no host
 * synchronisation) and overlaps the streaming of the following ops.
 *   n_allreduce_ops, max_allreduce_rows   how many ops of the plan have
 *               allreduce = 1 and their largest M
 *   peer_inbox  HOST array of `world` device pointers: rank p's inbox, at least
 *               feather_gemv_chain_inbox_floats(...) floats, 16-byte aligned,
 *               zero before the first call, as mapped into THIS process
 *   peer_flags  HOST array of `world` device pointers to the ranks' flag
 *               blocks (32 words, zero before the first call); this rank's own
 *               block holds the call counter, so a captured graph of launches
 *               may be replayed
 * Every rank launches the same table shape (same ops in the same order).  Waits
 * for the peers are bounded (feather_set_wait_limit_ms, feather_device_status).
 * An inbox and flag block serve ONE plan (or plans launched in the same order
 * on every rank).
 */
int64_t feather_gemv_chain_inbox_floats(int32_t n_allreduce_ops, int32_t max_allreduce_rows, int world);
int feather_gemv_chain_fp8_tp(const void* plan, int32_t n_ops, uint32_t flags, int32_t n_allreduce_ops,
                              int32_t max_allreduce_rows, float* const* peer_inbox, int64_t inbox_floats,
                              uint32_t* const* peer_flags, int rank, int world, void* stream);

/*
 * Kernel-variant knobs for A/B runs in benchmarks; results do not depend on
 * them.  No counterpart in the reference, whose only tunables are the
 * BLOCK_SIZE constants in its launch wrappers (feather/routines/gemv.py:178,
 * :229, feather/routines/dot.py:256).  `spec` is "key=value[,key=value...]":
 *   ring_pre_kb=K       KiB of each CTA's first rows that the large-matrix GEMV
 *                       kernel asks L2 for ahead of its stream-order wait, E5M2
 *                       (0 .. 16384, default 128; 0 = none)
 *   ring_pre_kb_e4m3=K  the same for E4M3 (-1 = by matrix size, the default)
 *   rows_pre=0|1        the same for the first batch of the small-matrix kernel
 *   dot_ring=0..3       0: the register-load dot kernel only; 1, 2, 3: long
 *                       operands take the bulk-copy ring kernel with stages of
 *                       32, 64 or 16 KiB
 *   dot_pre_kb=K        as ring_pre_kb, for the dot ring kernel
 *   dot_unroll=1|2|4    16-byte loads per operand a dot thread keeps in flight
 *   dot_ctas_per_sm=C   dot grid in CTAs per SM (1 .. 16)
 *   multi_tc=0|1        E5M2 GEMV against several vectors, large matrices with rows of
 *                       a multiple of 512 codes: 1 (default) the tcgen05 kernel, 16
 *                       vectors per pass; 0 the mma.sync kernel, 8 per pass
 *   attn_tc=0|1|2       attention on rows of 32 .. 512 codes: 0 the register-fed
 *                       mma.sync kernel, 1 (default) the tcgen05 kernel from 1024 /
 *                       1024 / 256 / 128 / 128 queries up, 2 the tcgen05 kernel for
 *                       every length
 * The environment variable FEATHER_KERNEL, if set, is applied once with the
 * same syntax when the library first touches a device.  Process-wide, takes
 * effect for later launches.  FEATHER_ERR_BAD_ARG for an unknown key or value;
 * keys before the offending one have been applied.
 */
int feather_set_tuning(const char* spec);

/*
 * *out = sum_i decode(a[i]) * decode(b[i]) over 4 * n_words codes.
 * Replaces feather/routines/dot.py:220-260 (dot_fp8_e5m2_acc_fp32_gpu) and its
 * kernel dot.py:144-192.  The reference adds per-block sums with a float
 * atomic (run-to-run different in the last bits); this one reduces in a fixed
 * order through `workspace`, so it is deterministic.  mode E4M3 (kernel decode
 * of gemv.py:83-88) is an extension: the reference has no E4M3 dot.
 *   workspace   feather_dot_workspace_bytes(n_words) bytes, 16-byte aligned.
 *               Its first 16 bytes must be zero before the FIRST use; the
 *               kernel leaves them zero again, so the buffer can be reused by
 *               later calls on the same stream without clearing.
 *   out         one float (written)
 */
int feather_dot_fp8(const uint32_t* a, const uint32_t* b, float* out, void* workspace,
                    int64_t n_words, int mode, void* stream);
int64_t feather_dot_workspace_bytes(int64_t n_words);

/*
 * feather_dot_fp8 for callers that cannot hand over a workspace because they
 * cannot allocate device memory at all.  It has no counterpart in the
 * reference.  Such callers exist: code that runs from a host callback queued
 * on a stream (the CUDA runtime forbids allocation calls there), a plug-in
 * inside a serving process whose device memory was given whole to another
 * allocator at start-up, or a latency-critical loop that must not take
 * cudaMalloc's device-wide synchronisation.  For them the scratch the kernel
 * needs (a ticket counter and one partial sum per CTA, about 4 KiB) is a fixed
 * array inside the library image instead of an argument; this call performs no
 * cudaMalloc, cudaFree or any other allocating routine.
 *
 *   a, b, out, n_words, mode, stream   as feather_dot_fp8
 *   limit    n_words <= feather_dot_fp8_static_max_words() (2^28 words, i.e.
 *            1 GiB of codes per operand); larger sizes return
 *            FEATHER_ERR_TOO_LARGE and launch nothing
 *
 * The array costs every GPU that loads the library those few KiB until the
 * process exits.  The first call on a device looks up the array's device
 * address (once per device); make that first call outside any stream capture.
 * All calls on a device share the one array: it still holds what the previous
 * call left (the call clears the part that must start at zero itself), and two
 * calls that can overlap on the GPU (different streams, no ordering between
 * them) race on it.  Serialise them, or use feather_dot_fp8 with one
 * workspace per stream.
 */
int feather_dot_fp8_static(const uint32_t* a, const uint32_t* b, float* out, int64_t n_words,
                           int mode, void* stream);
int64_t feather_dot_fp8_static_max_words(void);

#ifdef __cplusplus
}
#endif
#endif /* FEATHER_B200_H */
