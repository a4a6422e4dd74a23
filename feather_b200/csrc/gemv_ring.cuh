// gemv_ring_kernel: the packed-FP8 GEMV as a bulk-async-copy ring (sm_100a).
//
//   out[r] = sum_j decode(m[r, j]) * decode(v[j])     FP32 accumulation
//   (reference kernels: feather/routines/gemv.py:8-61 and :91-133)
//
// Why a ring: the kernel is HBM-bound, and B200 needs >40 KB of loads in flight
// per SM all the time to keep HBM3e busy.  Register-held loads tie that amount
// to occupancy and drain at every reduction.  Here one producer warp keeps a
// ring of STAGES shared-memory stages full with cp.async.bulk (the TMA engine's
// 1-D bulk copy, completion counted on an mbarrier), so ~190 KB per SM are in
// flight regardless of what the consumer warps are doing.
//
// Work split
//   * persistent grid, one CTA per SM; CTA b owns the contiguous rows
//     [M*b/G, M*(b+1)/G) and walks them in tasks of CW*RW rows;
//   * a stage holds, for every row of the task, the same SEGB = CL*512 bytes
//     of columns (one bulk copy per row and stage, issued by the lanes of the
//     producer warp in parallel); the walk is tasks, then column segments;
//   * consumer warp w OWNS rows w*RW .. w*RW+RW-1 of the task for all columns,
//     so a row's sum never leaves the warp: no CTA-wide barrier in the loop,
//     only mbarrier waits, and one shuffle butterfly per task;
//   * the vector lives in shared memory as FP16 pairs (the decoded values of
//     both formats are FP16 numbers) in a layout whose 128-bit reads are
//     conflict-free.  Up to 16384 codes it is decoded once per CTA; longer
//     vectors are cut into pieces of 8192 codes that alternate between two
//     buffers, staged by a dedicated warp one piece ahead of the consumers;
//     partial row sums between pieces stay in shared memory;
//   * matrix codes are decoded in registers to FP16 pairs (fp8_codec.cuh) and
//     multiplied with the mixed-precision FMA fma.rn.f32.f16 (FP16 operands,
//     FP32 accumulator, one rounding): the product of two FP16 numbers is
//     exact in FP32, so this equals the reference's convert-then-multiply.
//
// Every wait is bounded: after kWaitLimitNs without progress a thread raises
// the status word and stops waiting; the host reads the word with
// feather_device_status().  Every copy has exactly one destination CTA.
#pragma once
#include "gemv_common.cuh"

namespace feather {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises *status) if the phase did not
// complete within kWaitLimitNs.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int* status) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > kWaitLimitNs) {
            atomicOr(status, 1u);
            return false;
        }
    }
}
// The same bounded wait for kernels whose waiting warps would otherwise starve the
// warps they wait for: a warp that polls an mbarrier in a tight loop takes issue slots,
// and with 16 consumer warps polling, a producer warp that has real work to do per step
// (the table walk of the chain kernel) gets a nineteenth of its SM sub-partition's issue
// bandwidth -- measured as a floor of half a microsecond per GEMV however small.  Here
// the waiter sleeps a few tens of nanoseconds between looks.
__device__ __forceinline__ bool mbar_wait_backoff(uint32_t bar, uint32_t parity, unsigned int* status,
                                                  unsigned int sleep_ns = 40) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i) {
            __nanosleep(sleep_ns);
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (global_timer_ns() - t0 > kWaitLimitNs) {
            atomicOr(status, 1u);
            return false;
        }
    }
}
// 1-D bulk copy global -> this CTA's shared memory, completion on `bar`.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Barrier over the threads counted by `bar` (arrive, then a bounded wait).
__device__ __forceinline__ bool mbar_sync(uint32_t bar, uint32_t& parity, unsigned int* status) {
    mbar_arrive(bar);
    const bool ok = mbar_wait(bar, parity, status);
    parity ^= 1u;
    return ok;
}

#ifdef FEATHER_RING_STAMPS
// Diagnostic build only (-DFEATHER_RING_STAMPS): the GPU's nanosecond timer at six
// points of every CTA of gemv_ring_kernel, for the 16 most recent launches (the slot is
// taken from the output address, so give consecutive launches outputs 64 KiB apart):
// [0] entry, [1] past the stream-order wait, [2] first stage issued, [3] first stage
// landed, [4] vector staged, [5] last row written.  Read with feather_debug_ring_stamps.
__device__ unsigned long long g_ring_stamps[16][160][8];
#define RING_STAMP(out_ptr, i)                                                                         \
    g_ring_stamps[(reinterpret_cast<uintptr_t>(out_ptr) >> 16) & 15][blockIdx.x < 160 ? blockIdx.x : 159][i] = \
        global_timer_ns()
#else
#define RING_STAMP(out_ptr, i) ((void)0)
#endif

// Row-sharded multi-GPU launch (FUSED = true): where every rank's output
// buffer and flag block live.  Pointers are valid on THIS device (peer-mapped).
constexpr int kMaxShardRanks = 16;
constexpr int kShardStageRows = 512;  // results a CTA can stage in shared memory before pushing
constexpr int kShardTicketWord = kMaxShardRanks;  // flag-block word used as this rank's CTA ticket
struct ShardArgs {
    float* out[kMaxShardRanks];          // rank p's full output buffer
    unsigned int* flags[kMaxShardRanks]; // rank p's flag block: word q = last epoch rank q delivered
    long long row_offset;                // first global row of this rank's block
    int rank, world;
    unsigned int epoch;                  // this call's number, increasing by one per call
    int staged;                          // 1: every CTA owns <= kShardStageRows rows; a dedicated warp
                                         //    pushes each task's rows to the peers, coalesced, as soon
                                         //    as the task is done;
                                         // 0: each row is stored to the peers as it finishes
    int no_wait;                         // 1: the kernel ends once its rows and its epoch are on their
                                         //    way; the caller waits for the peers' epochs separately
    unsigned long long* stamps;          // optional (may be null): %globaltimer of the rank's last CTA
                                         //    [0] rows pushed, [1] epoch published, [2] all epochs seen
};
template <int CW, int RW, int CL, int STAGES, int TILE>
struct RingGeometry {
    static constexpr int kTaskRows = CW * RW;          // rows per task (= per stage)
    static constexpr int kSegChunks = CL * 32;         // 16-byte chunks per row and stage
    static constexpr int kSegBytes = kSegChunks * 16;
    static constexpr int kStageBytes = kTaskRows * kSegBytes;
    static constexpr int kTileChunks = TILE / 16;      // vector chunks resident when N <= TILE
    static constexpr int kHalfChunks = kTileChunks / 2;  // per buffer when the vector is longer
    static constexpr int kVecBytes = TILE * 2;         // FP16 vector region (one tile or two halves)
    // mbarriers: full[STAGES], empty[STAGES], start, vec_full[2], vec_empty[2]; then one counter word
    static constexpr int kBarriers = 2 * STAGES + 5;
    static constexpr int kMaxTasks = 64;               // per-task arrival counters of a fused launch
    static constexpr int kSmemBytes = kVecBytes + STAGES * kStageBytes + (kBarriers + 1) * 8 +
                                      kShardStageRows * 4 + kMaxTasks * 4;
    static constexpr int kThreads = (CW + 2) * 32;     // consumers, producer warp, vector warp
    static constexpr int kThreadsFused = (CW + 3) * 32;  // + the exchange warp of a row-sharded launch
    static_assert(kHalfChunks % kSegChunks == 0, "a vector half holds whole segments");
};

// Stage `n_chunks` chunks (16 codes each) of the packed vector, starting at word
// `v`, into `dst` as FP16 pairs: (group g, half k, lane l) is the uint4 at
// (g*2 + k)*32 + l and holds codes 16*(32g+l) + 8k .. +7.  Chunks from n_chunks
// up to `fill_chunks` are written as zero codes.  Called by `n_threads` threads
// with ids `tid`; BATCH loads are in flight per thread (the loads come from L2,
// so a single warp needs a deep batch to stage a piece in about a microsecond).
template <int MODE, int BATCH>
__device__ __forceinline__ void stage_vector(uint4* dst, const uint32_t* __restrict__ v,
                                             int n_chunks, int fill_chunks, int tid, int n_threads) {
    uint2* vec2 = reinterpret_cast<uint2*>(dst);
    const int w_valid = n_chunks * 4, w_fill = fill_chunks * 4;
    constexpr int kBatch = BATCH;
    for (int w0 = tid; w0 < w_fill; w0 += kBatch * n_threads) {
        uint32_t raw[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int wl = w0 + b * n_threads;
            raw[b] = wl < w_valid && bounds_ok(wl >= 0) ? __ldg(v + wl) : 0u;  // beyond N: code 0 = +0.0
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int wl = w0 + b * n_threads;
            if (wl < w_fill) {
                uint32_t lo, hi;
                decode_word_h2<MODE>(raw[b], lo, hi);
                const int chunk = wl >> 2, k = wl & 3;
                vec2[(((chunk >> 5) * 2 + (k >> 1)) * 32 + (chunk & 31)) * 2 + (k & 1)] = make_uint2(lo, hi);
            }
        }
    }
}

// The walk every role follows: vector pieces outermost, then the tasks (row
// groups of the CTA), then the 4 KiB segments of the piece.
//   short rows (N <= TILE): one piece, the whole vector, staged once by the
//     consumer warps;
//   long rows: pieces of TILE/2 codes that alternate between the two halves of
//     the vector region; a dedicated warp stages piece p+1 while the consumers
//     use piece p, so the stream never drains at a piece boundary.  Partial row
//     sums between pieces stay in shared memory.
//
// CTAS: CTAs resident per SM the launch is sized for.  PREFETCH: the producer
// also asks L2 for the next task's rows (cp.async.bulk.prefetch.L2); measured
// slower and left off.
// FUSED: the kernel is one rank of a row-sharded GEMV.  Finished rows are
// stored straight into EVERY rank's output buffer (plain stores to peer-mapped
// memory over NVLink), so the gather of the output slices happens inside the
// GEMV instead of in a separate collective.  An extra warp does the exchange:
// it waits (shared-memory counters) for each task's rows, pushes them to all
// ranks as coalesced 64-byte runs while the consumers go on with the next
// task, and at the end takes the rank's CTA ticket.  The last CTA of the rank
// publishes the call's epoch in every rank's flag block.  Before the first
// push of call e the exchange warp makes sure every peer has delivered call
// e - 1: a peer that has delivered e - 1 has been launched for it, so the
// result of call e - 2 in the buffer about to be overwritten (two buffers
// alternate by epoch parity) is no longer wanted -- a result is valid until the
// rank's next call.  Then either the last CTA waits (bounded) until all ranks'
// epochs have arrived here, so that the buffer holds the full result when the
// kernel ends, or (sh.no_wait) it returns and the caller waits separately
// (shard_wait_kernel) before it reads the result: the exchange latency and the
// skew between ranks then overlap the next call instead of ending every call.
// EARLY: the caller promises that nothing earlier in the stream writes the
// MATRIX (static weights).  The producer warp then starts streaming matrix
// bytes before the stream-order wait, so a kernel that was launched early
// (programmatic dependent launch) fills its ring while its predecessor still
// drains; the vector is read and the output written only after the wait.
template <int MODE, int CW, int RW, int CL, int STAGES, int TILE, int CTAS, bool PREFETCH,
          bool FUSED = false, bool EARLY = false>
__global__ void __launch_bounds__((CW + 2 + (FUSED ? 1 : 0)) * 32, CTAS)
gemv_ring_kernel(const unsigned char* __restrict__ m, const uint32_t* __restrict__ v,
                 float* __restrict__ out, int M, int n16, unsigned int* __restrict__ status,
                 int pre_bytes, const __grid_constant__ ShardArgs sh = ShardArgs{}) {
    using G = RingGeometry<CW, RW, CL, STAGES, TILE>;
    // Programmatic dependent launch: let the next kernel of the stream be
    // scheduled onto SMs as they free up.  Everything up to the stream-order
    // wait below touches no global memory, so it runs under the tail of the
    // kernel before this one.  Without the launch attribute both are no-ops.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) RING_STAMP(out, 0);
    extern __shared__ __align__(128) unsigned char smem[];
    uint4* vec = reinterpret_cast<uint4*>(smem);
    unsigned char* ring = smem + G::kVecBytes;
    const uint32_t ring_s = smem_u32(ring);
    unsigned char* bar_mem = ring + STAGES * G::kStageBytes;
    const uint32_t bars = smem_u32(bar_mem);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t start_bar = bars + 8u * (2 * STAGES);       // all consumer threads
    auto vec_full = [&](int b) { return bars + 8u * (2 * STAGES + 1 + b); };
    auto vec_empty = [&](int b) { return bars + 8u * (2 * STAGES + 3 + b); };
    unsigned int* warps_done = reinterpret_cast<unsigned int*>(bar_mem + 8 * G::kBarriers);
    float* staged_rows = reinterpret_cast<float*>(bar_mem + 8 * (G::kBarriers + 1));
    unsigned int* task_cnt = reinterpret_cast<unsigned int*>(staged_rows + kShardStageRows);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row_begin = (int)(((long long)M * blockIdx.x) / gridDim.x);
    const int row_end = (int)(((long long)M * (blockIdx.x + 1)) / gridDim.x);
    const int n_tasks = (row_end - row_begin + G::kTaskRows - 1) / G::kTaskRows;
    // Rows per task.  E5M2 is bound by the bytes in flight, so its rows are
    // balanced over the tasks: 55 rows are walked as 14+14+14+13, not 16+16+16+7,
    // and no stage of the ring is mostly empty.  E4M3 is bound by instruction
    // issue and keeps every consumer warp busy instead (full tasks, one short).
    const int task_rows = (MODE == kE5M2 && n_tasks > 0)
        ? ((row_end - row_begin + n_tasks * RW - 1) / (n_tasks * RW)) * RW : G::kTaskRows;
    const size_t row_bytes = (size_t)n16 * 16;
    const bool long_rows = n16 > G::kTileChunks;
    const int piece_chunks = long_rows ? G::kHalfChunks : G::kTileChunks;  // vector chunks per piece
    const int n_pieces = (n16 + piece_chunks - 1) / piece_chunks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);     // the producer's arrive + the copied bytes
            mbar_init(empty_bar(s), CW);   // one arrive per consumer warp
        }
        mbar_init(start_bar, CW * 32);
        for (int b = 0; b < 2; ++b) {
            mbar_init(vec_full(b), 1);     // the vector warp, once the piece is staged
            mbar_init(vec_empty(b), CW);   // one arrive per consumer warp
        }
        *warps_done = 0u;
        if (FUSED)
            for (int t = 0; t < G::kMaxTasks; ++t) task_cnt[t] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (!EARLY && warp == CW && pre_bytes > 0) {
        // Ahead of the stream-order wait the producer asks L2 for the first
        // `pre_bytes` of this CTA's rows.  A prefetch only moves lines from HBM
        // into L2, the point where all writes to this GPU's memory meet, so it
        // is harmless even when the kernel before this one is still writing
        // the matrix: the copies issued after the wait read what L2 then holds.
        // CTAs of a kernel launched back to back land on SMs as the previous
        // kernel's CTAs retire, and these requests fill the HBM time its tail
        // leaves idle.
        const int chunks_p0 = min(piece_chunks, n16);
        const int pre_rows = min(row_end - row_begin, (pre_bytes + chunks_p0 * 16 - 1) / (chunks_p0 * 16));
        for (int r = lane; r < pre_rows; r += 32)
            bulk_prefetch_l2(m + (size_t)(row_begin + r) * row_bytes, (uint32_t)chunks_p0 * 16u);
    }
    __syncthreads();
    if (!EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) RING_STAMP(out, 1);
    if (n_tasks == 0 && !FUSED) return;  // a fused rank needs every CTA at the final ticket

    if (FUSED && warp == CW + 2) {
        // -------------------------------------------------- exchange warp --
        if (EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");  // it writes the outputs
        unsigned int* my_flags = sh.flags[sh.rank];
        if (sh.staged && n_tasks > 0) {
            // every peer must have delivered the call before this one (see above)
            if (lane < sh.world) {
                const unsigned int need = sh.epoch - 1u;
                if ((int)(ld_relaxed_sys(my_flags + lane) - need) < 0) {
                    const unsigned long long t0 = global_timer_ns();
                    while ((int)(ld_relaxed_sys(my_flags + lane) - need) < 0) {
                        if (global_timer_ns() - t0 > kWaitLimitNs) {
                            atomicOr(status, 2u);  // rank `lane` never delivered the previous call
                            break;
                        }
                    }
                }
            }
            __syncwarp();
            bool alive = true;
            for (int task = 0; task < n_tasks && alive; ++task) {
                const int t_row0 = task * task_rows;                       // CTA-local
                const int t_rows = min(task_rows, row_end - row_begin - t_row0);
                // the consumers count every finished row of the task in task_cnt[task]
                const volatile unsigned int* cnt = task_cnt + task;
                if (*cnt < (unsigned int)t_rows) {
                    const unsigned long long t0 = global_timer_ns();
                    while (*cnt < (unsigned int)t_rows) {
                        __nanosleep(64);
                        if (global_timer_ns() - t0 > kWaitLimitNs) {
                            atomicOr(status, 1u);
                            alive = false;
                            break;
                        }
                    }
                }
                __threadfence_block();   // the rows counted above are visible to this warp
                if (!alive) break;
                // two ranks per pass: lanes 0-15 and 16-31 each store one 64-byte run
                const int i = lane & 15;
                for (int k = 0; k < sh.world; k += 2) {
                    const int kk = k + (lane >> 4);
                    if (kk < sh.world && i < t_rows && bounds_ok(row_begin + t_row0 + i < M)) {
                        const int p = (sh.rank + kk) % sh.world;  // own buffer first, then round the ring
                        sh.out[p][sh.row_offset + row_begin + t_row0 + i] = staged_rows[t_row0 + i];
                    }
                }
            }
        }
        // All rows of this CTA are on their way (staged mode) or were stored by the consumers:
        // wait for the consumers' count in the other mode, then take the rank's ticket.
        if (!sh.staged) {
            const volatile unsigned int* cnt = warps_done;
            const unsigned long long t0 = global_timer_ns();
            while (*cnt < (unsigned int)CW) {
                __nanosleep(64);
                if (global_timer_ns() - t0 > kWaitLimitNs) {
                    atomicOr(status, 1u);
                    break;
                }
            }
        }
        __syncwarp();
        __threadfence_system();  // the pushed rows are visible everywhere before the ticket
        unsigned int ticket = 0;
        if (lane == 0) ticket = atomicAdd(my_flags + kShardTicketWord, 1u);
        ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
        if (ticket == gridDim.x - 1) {
            // last CTA of this rank: lane q tells rank q "my slice is with you"
            if (lane == 0) {
                my_flags[kShardTicketWord] = 0u;  // ready for the next call
                if (sh.stamps) sh.stamps[0] = global_timer_ns();
            }
            __threadfence_system();
            if (lane < sh.world) st_relaxed_sys(sh.flags[lane] + sh.rank, sh.epoch);
            if (lane == 0 && sh.stamps) sh.stamps[1] = global_timer_ns();
            if (!sh.no_wait) {
                // ... and waits for rank q's slice here -- all peers in parallel
                if (lane < sh.world) {
                    const unsigned long long t0 = global_timer_ns();
                    // wrap-safe "flag has reached this epoch"
                    while ((int)(ld_relaxed_sys(my_flags + lane) - sh.epoch) < 0) {
                        if (global_timer_ns() - t0 > kWaitLimitNs) {
                            atomicOr(status, 2u);  // rank `lane`'s slice did not arrive in time
                            break;
                        }
                    }
                }
                __syncwarp();
                __threadfence_system();  // the peers' rows are visible to whatever runs next
                if (lane == 0 && sh.stamps) sh.stamps[2] = global_timer_ns();
            }
        }
        return;
    }

    if (warp == CW + 1) {
        // ---------------------------------------------------- vector warp --
        if (!long_rows) return;
        if (EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");  // it reads the vector
        for (int piece = 0; piece < n_pieces; ++piece) {
            const int b = piece & 1;  // pieces alternate between the two halves
            // the half is free once the consumers are done with piece - 2
            if (piece >= 2 && !mbar_wait(vec_empty(b), (uint32_t)((piece >> 1) - 1) & 1u, status)) return;
            const int chunks = min(piece_chunks, n16 - piece * piece_chunks);
            const int fill = ((chunks + G::kSegChunks - 1) / G::kSegChunks) * G::kSegChunks;
            stage_vector<MODE, 8>(vec + b * (G::kHalfChunks * 2), v + (size_t)piece * piece_chunks * 4,
                                   chunks, fill, lane, 32);
            __syncwarp();
            if (lane == 0) mbar_arrive(vec_full(b));
        }
        return;
    }

    if (warp == CW) {
        // ------------------------------------------------------- producer --
        if (lane == 0) RING_STAMP(out, 6);
        int s = 0;               // ring slot of the next stage
        uint32_t round = 0;      // how many times the ring has wrapped
        bool alive = true;
        for (int piece = 0; piece < n_pieces && alive; ++piece) {
            const int chunks_p = min(piece_chunks, n16 - piece * piece_chunks);
            const int n_seg = (chunks_p + G::kSegChunks - 1) / G::kSegChunks;
            for (int task = 0; task < n_tasks && alive; ++task) {
                const int row0 = row_begin + task * task_rows;
                const int valid_rows = min(task_rows, row_end - row0);
                if (PREFETCH && task + 1 < n_tasks) {
                    const int p_rows = min(task_rows, row_end - row0 - task_rows);
                    for (int r = lane; r < p_rows; r += 32)
                        bulk_prefetch_l2(m + (size_t)(row0 + task_rows + r) * row_bytes +
                                             (size_t)piece * piece_chunks * 16,
                                         (uint32_t)chunks_p * 16u);
                }
                for (int seg = 0; seg < n_seg; ++seg) {
                    if (round > 0 && !mbar_wait(empty_bar(s), (round & 1u) ^ 1u, status)) {
                        alive = false;
                        break;
                    }
                    const int chunks = min(G::kSegChunks, chunks_p - seg * G::kSegChunks);
                    const uint32_t bytes = (uint32_t)chunks * 16u;
                    if (lane == 0) mbar_arrive_expect_tx(full_bar(s), bytes * (uint32_t)valid_rows);
                    const size_t col = ((size_t)piece * piece_chunks + (size_t)seg * G::kSegChunks) * 16;
                    for (int r = lane; r < valid_rows; r += 32)
                        if (bounds_ok(row0 + r < M && col + bytes <= row_bytes && r < G::kTaskRows))
                            bulk_load(ring_s + s * G::kStageBytes + r * G::kSegBytes,
                                      m + (size_t)(row0 + r) * row_bytes + col, bytes, full_bar(s));
                    if (piece == 0 && task == 0 && seg == 0 && lane == 0) RING_STAMP(out, 2);
                    if (++s == STAGES) { s = 0; ++round; }
                }
            }
        }
        if (!alive) {
            // a wait gave up: give the copies already issued time to land
            // before the CTA's shared memory is released
            const unsigned long long t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 1000000ull) {}
        }
        return;
    }

    // ---------------------------------------------------------- consumers --
    if (EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");  // before the vector and the output
    int s = 0;            // ring slot of the next stage
    uint32_t phase = 0;   // its mbarrier parity
    bool alive = true;
    const uint4* const ring_lane = reinterpret_cast<const uint4*>(ring) + (warp * RW) * G::kSegChunks + lane;
    if (!long_rows) {
        // the whole vector, once, by all consumer warps
        const int fill = ((n16 + G::kSegChunks - 1) / G::kSegChunks) * G::kSegChunks;
        stage_vector<MODE, 4>(vec, v, n16, fill, threadIdx.x, CW * 32);
        uint32_t parity = 0;
        alive = mbar_sync(start_bar, parity, status);
        if (threadIdx.x == 0) RING_STAMP(out, 4);
    }
    // Partial row sums between pieces: in shared memory when the CTA's row block
    // fits there (no global round trip in the loop), else in the output buffer.
    const bool smem_acc = row_end - row_begin <= kShardStageRows;
    float* const partial = FUSED ? sh.out[sh.rank] + sh.row_offset : out;
    for (int piece = 0; piece < n_pieces && alive; ++piece) {
        const int chunks_p = min(piece_chunks, n16 - piece * piece_chunks);
        const int n_seg = (chunks_p + G::kSegChunks - 1) / G::kSegChunks;
        const int n_full_seg = chunks_p / G::kSegChunks;
        const bool last_piece = piece + 1 == n_pieces;
        const uint4* vbase = vec;
        if (long_rows) {
            const int b = piece & 1;
            vbase = vec + b * (G::kHalfChunks * 2);
            if (!mbar_wait(vec_full(b), (uint32_t)(piece >> 1) & 1u, status)) break;
        }
        for (int task = 0; task < n_tasks && alive; ++task) {
            const int task_end = min(row_end, row_begin + (task + 1) * task_rows);
            const int row0 = row_begin + task * task_rows + warp * RW;
            const bool all_rows = row0 + RW <= task_end;  // warp-uniform
            float acc[RW][4];
#pragma unroll
            for (int r = 0; r < RW; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;

            for (int seg = 0; seg < n_seg; ++seg) {
                if (!mbar_wait(full_bar(s), phase, status)) {
                    alive = false;
                    break;
                }
                if (threadIdx.x == 0 && piece == 0 && task == 0 && seg == 0) RING_STAMP(out, 3);
                const uint4* st = ring_lane + s * (G::kStageBytes / 16);
                const uint4* vs = vbase + (seg * CL * 2) * 32 + lane;
                if (all_rows && seg < n_full_seg) {
                    // whole segment, all rows: no predicates, fully unrolled
#pragma unroll
                    for (int c = 0; c < CL; ++c) {
                        const uint4 va = vs[(c * 2) * 32], vb = vs[(c * 2 + 1) * 32];
#pragma unroll
                        for (int r = 0; r < RW; ++r)
                            fma_chunk<MODE>(st[r * G::kSegChunks + c * 32], va, vb, acc[r]);
                    }
                } else {
                    const int chunks = min(G::kSegChunks, chunks_p - seg * G::kSegChunks);
#pragma unroll 1
                    for (int c = 0; c < CL; ++c) {
                        if (c * 32 + lane < chunks) {
                            const uint4 va = vs[(c * 2) * 32], vb = vs[(c * 2 + 1) * 32];
#pragma unroll
                            for (int r = 0; r < RW; ++r)
                                if (row0 + r < task_end)
                                    fma_chunk<MODE>(st[r * G::kSegChunks + c * 32], va, vb, acc[r]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(s));  // this warp is done with the stage
                if (++s == STAGES) { s = 0; phase ^= 1u; }
            }
            if (!alive) break;
            // the warp owns its rows: one butterfly, then the row's lane adds the
            // earlier pieces' partial sum and writes
            float sums[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) sums[r] = (acc[r][0] + acc[r][1]) + (acc[r][2] + acc[r][3]);
            warp_reduce_rows<RW>(sums, lane);
            if ((lane & (32 / RW - 1)) == 0) {
                const int row = row0 + lane / (32 / RW);
                if (row < task_end) {
                    float total = sums[0];
                    if (piece > 0) total += smem_acc ? staged_rows[row - row_begin] : partial[row];
                    if (!last_piece) {
                        if (smem_acc) staged_rows[row - row_begin] = total;
                        else partial[row] = total;  // the same lane owns the row in every piece
                    } else if (!FUSED) {
                        if (bounds_ok(row >= 0 && row < M)) out[row] = total;
                    } else if (sh.staged) {
                        // the exchange warp pushes the task's rows once all of them are here
                        staged_rows[row - row_begin] = total;
                        __threadfence_block();
                        atomicAdd(task_cnt + task, 1u);
                    } else {
                        for (int p = 0; p < sh.world; ++p) sh.out[p][sh.row_offset + row] = total;
                        __threadfence_system();  // before this warp reports itself finished
                    }
                }
            }
        }
        if (!alive) break;
        if (long_rows) {
            __syncwarp();
            if (lane == 0) mbar_arrive(vec_empty(piece & 1));  // this warp is done with the piece
        }
    }
    if (threadIdx.x == 0) RING_STAMP(out, 5);
    if (FUSED && !sh.staged) {
        // rows went to the peers one by one: tell the exchange warp this warp is done
        __syncwarp();
        if (lane == 0) atomicAdd(warps_done, 1u);
    }
}

// Second half of a split-phase row-sharded call (sh.no_wait): returns once every
// rank's epoch has reached `epoch` in this rank's flag block, i.e. once all
// slices of that call sit in this rank's output buffer.  One warp; bounded.
__global__ void __launch_bounds__(32)
shard_wait_kernel(const unsigned int* __restrict__ my_flags, int world, unsigned int epoch,
                  unsigned int* __restrict__ status, unsigned long long* __restrict__ stamps) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x;
    if (lane < world) {
        const unsigned long long t0 = global_timer_ns();
        while ((int)(ld_relaxed_sys(my_flags + lane) - epoch) < 0) {
            if (global_timer_ns() - t0 > kWaitLimitNs) {
                atomicOr(status, 2u);
                break;
            }
        }
    }
    __syncwarp();
    __threadfence_system();
    if (lane == 0 && stamps) stamps[2] = global_timer_ns();
}

}  // namespace feather
