// gemv_chain_kernel: a whole table of packed-FP8 GEMVs in ONE persistent launch.
//
//   for every op i of the table:  out_i[r] = sum_j decode(m_i[r, j]) * decode(v_i[j])
//
// Batch-1 decoding runs a chain of small GEMVs (a TinyLlama-shaped token is 155
// of them, 0.5 .. 65 MB each).  Launched one by one they are bound by launch
// and prologue latency, not by HBM: every kernel starts with an empty pipeline
// and ends by draining it.  Here the grid (one CTA per SM) walks the table and
// the stream of matrix bytes never stops at an op boundary:
//
//   * the producer warp walks (op, task, segment) and keeps a ring of
//     kChainStages shared-memory stages full with cp.async.bulk; a stage holds
//     up to 16 rows x 2 KiB of one op (rows of one segment as a few large
//     copies: the copy engine charges per request); it runs ahead across op
//     boundaries as far as the ring allows (weights do not depend on earlier ops);
//   * 16 consumer warps each OWN one row of a stage for all its columns (no
//     CTA-wide reduction; the arithmetic and its order are those of
//     gemv_rows_kernel / gemv_ring_kernel, so every op's result has the bits
//     of the single-op entry point);
//   * the vector warp stages the NEXT op's vector (decoded once to FP16 pairs,
//     two buffers) while the consumers still work on the current op; ops that
//     share a vector (q/k/v, gate/up) and wait for the same op, or for none,
//     stage it once;
//   * an op may name an earlier op it depends on (`wait_op`: its vector is that
//     op's packed output).  CTAs that finish their rows of an op count
//     themselves in done[op] (release); the vector warp of a dependent op polls
//     that counter (acquire, bounded) before it reads the vector with L2 loads.
//     The matrix stream is not held up by such a wait until the ring is full;
//   * results are FP32 sums or, with out_mode >= 0, FP8 codes of the sums (the
//     packer's rounding) stored one byte per row -- the packed vector the next
//     op consumes;
//   * tensor-parallel launches (one per GPU): an op may be COLUMN-sharded, every
//     rank holding a column block of all rows and the matching slice of the
//     vector.  Its row sums are partial: a task's sums meet in shared memory
//     and go, as (sum, call number) pairs, into every rank's inbox through
//     peer-mapped pointers -- eight bytes that arrive whole, so the data is its
//     own arrival flag, 128 contiguous bytes per rank and task -- and the
//     consumers go on with the next task.  A further warp, the reduce warp,
//     reads this rank's inbox for the pairs of all ranks (polling, bounded, what
//     has not arrived), adds them in rank order and writes the result: the same
//     bits on every rank, no collective launch, and the NVLink round trip
//     overlaps the streaming of the following ops.
//     Every all-reduced op of a launch has its own inbox region, and two sets
//     of regions alternate by the parity of the call number, which lives in
//     device memory so that a captured graph can be replayed.
//
// Rows of op i are dealt to the CTAs in contiguous blocks of whole 16-row tasks,
// rotated by the op index so that an uneven split does not always hit the same CTAs.
// The grid must be resident at once when ops depend on each other (checked by
// the host with the occupancy API).  Every wait is bounded (status word).
#pragma once
#include "gemv_ring.cuh"

namespace feather {

// One GEMV of the table as the kernel reads it (built by feather_gemv_chain_plan
// from the public feather_chain_op records; same size, 48 bytes).
struct ChainOp {
    const unsigned char* m;   // packed matrix, M rows of N bytes, 16-byte aligned rows
    const uint32_t* v;        // packed vector, N / 4 words, 16-byte aligned
    void* out;                // M floats, or ceil(M / 4) packed words when there is an output format
    int M, N;                 // N a multiple of 16, at most kChainTile
    int flags;                // bit 0: decode of m and v (kE5M2 / kE4M3); bits 1-2: 0 = FP32 sums,
                              // 1 + format = the sums encoded to that format; bit 3: a later op waits
                              // for this one; bits 4..: 0, or 1 + the op's index among the launch's
                              // all-reduced (column-sharded) ops
    int wait_op;              // -1, or the index of an EARLIER op that writes v
    int rows_q;               // ceil(M / 16) / grid: every CTA's share of the op's 16-row tasks; the
                              // first (tasks % grid) CTAs hold one more
    int rot;                  // (op index * kChainRotate) % grid: where the row blocks start
    __host__ __device__ int mode() const { return flags & 1; }
    __host__ __device__ int out_mode() const { return ((flags >> 1) & 3) - 1; }
    __host__ __device__ bool signal() const { return (flags & 8) != 0; }
    __host__ __device__ int ar_index() const { return (flags >> 4) - 1; }
};
static_assert(kE5M2 == 0 && kE4M3 == 1, "mode fits one bit");
static_assert(sizeof(ChainOp) == 48, "the table layout is part of the ABI");

constexpr int kChainCW = 16;                    // consumer warps = rows per stage
constexpr int kChainCL = 4;                     // 16-byte chunks per lane, row and stage
constexpr int kChainStages = 5;
constexpr int kChainCachedOps = 640;            // table entries kept in shared memory (the rest is read from global)
constexpr int kChainTile = 8192;                // longest row / vector, in codes
constexpr int kChainSegChunks = kChainCL * 32;  // 128 chunks = 2 KiB of a row per stage
constexpr int kChainSegBytes = kChainSegChunks * 16;
constexpr int kChainStageBytes = kChainCW * kChainSegBytes;       // 32 KiB
constexpr int kChainVecBytes = kChainTile * 2;                    // one FP16 vector buffer
constexpr int kChainBarriers = 2 * kChainStages + 4;              // full, empty, vec_full[2], vec_empty[2]
constexpr int kChainArSlots = 8;                 // tasks of an all-reduced op whose partial sums wait in shared memory
constexpr int kChainSmemBytes = 2 * kChainVecBytes + kChainStages * kChainStageBytes +
                                kChainBarriers * 8 + 8 * 4 +       // + 8 per-op arrival counters
                                kChainCachedOps * 48 +             // + the table
                                kChainArSlots * (kChainCW + 1) * 4;  // + partial sums and their counters
constexpr int kChainThreads = (kChainCW + 3) * 32;   // consumers, producer, vector warp, reduce warp

// Tensor-parallel launch: where every rank's inbox and flag block live, as mapped
// into this process (world = 0: a single-GPU launch).  Inbox layout, in 8-byte
// (sum, call number) pairs: [parity of the call][all-reduced op][source rank][row],
// `rows_cap` rows per source rank.
struct ChainArArgs {
    float* inbox[kMaxArRanks];
    unsigned int* flags[kMaxArRanks];   // only this rank's own is used (call counter, kArEpochWord)
    int rank, world;
    int n_ar;                           // all-reduced ops in the table
    int rows_cap;                       // rows per (op, source rank) slot
    __device__ size_t pair_index(unsigned int epoch, int ar, int src, int row) const {
        return ((((size_t)(epoch & 1u) * n_ar + ar) * world + src) * rows_cap + row);
    }
};
__device__ __forceinline__ void st_volatile_v2(float* p, uint32_t a, uint32_t b) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_volatile_v2(const float* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// The code (or float) of one finished row goes to its place in the op's output.
__device__ __forceinline__ void chain_store_row(const ChainOp& d, int row, float sum) {
    const int out_mode = d.out_mode();
    if (out_mode < 0) {
        reinterpret_cast<float*>(d.out)[row] = sum;
    } else {
        // one code per row, byte r of the packed output; the row that ends the matrix also
        // writes the zero codes that pad the last word
        unsigned char* codes = reinterpret_cast<unsigned char*>(d.out);
        codes[row] = (unsigned char)(out_mode == kE5M2 ? encode_f32<kE5M2>(sum) : encode_f32<kE4M3>(sum));
        if (row == d.M - 1)
            for (int i = d.M; i & 3; ++i) codes[i] = 0;
    }
}
constexpr int kChainRotate = 61;                // row blocks move by this many CTAs per op

struct ChainGeom {
    int row_begin, row_end, n_tasks, n16, n_seg;
};
__device__ __forceinline__ ChainGeom chain_geom(const ChainOp& d) {
    ChainGeom g;
    int b = (int)blockIdx.x + d.rot;
    if (b >= (int)gridDim.x) b -= (int)gridDim.x;
    // whole tasks of 16 rows are dealt out, not rows: a small op then fills the stages of a
    // few CTAs instead of putting one or two rows on every CTA, and the other CTAs pass it
    // at the cost of reading its table entry (the per-op bookkeeping of 19 warps is what a
    // small op costs; which CTAs pay it rotates with the op)
    const int tasks = (d.M + kChainCW - 1) / kChainCW;
    const int rem = tasks - d.rows_q * (int)gridDim.x;
    const int t_begin = b * d.rows_q + min(b, rem);
    g.n_tasks = d.rows_q + (b < rem ? 1 : 0);
    g.row_begin = t_begin * kChainCW;
    g.row_end = min(d.M, (t_begin + g.n_tasks) * kChainCW);
    g.n16 = d.N >> 4;
    g.n_seg = (g.n16 + kChainSegChunks - 1) / kChainSegChunks;
    return g;
}
// Table entry `op`: from the copy in shared memory (`cache`, the first kChainCachedOps
// entries) or from global memory; past the end the last op is read again (unused).
__device__ __forceinline__ ChainOp chain_load_op(const ChainOp* ops, const uint4* cache, int op, int n_ops) {
    if (op >= n_ops) op = n_ops - 1;
    union { uint4 q[3]; ChainOp d; } u;
    if (op < kChainCachedOps) {
        const uint4* p = cache + 3 * op;
        u.q[0] = p[0];
        u.q[1] = p[1];
        u.q[2] = p[2];
    } else {
        const uint4* p = reinterpret_cast<const uint4*>(ops + op);
        u.q[0] = __ldg(p);
        u.q[1] = __ldg(p + 1);
        u.q[2] = __ldg(p + 2);
    }
    return u.d;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_l2(const uint4* p) {
    uint4 r;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}

// One stage of one row: `chunks` 16-byte chunks (at most kChainSegChunks) of the
// row at `st` against the vector chunks at `vs`.
template <int MODE>
__device__ __forceinline__ void chain_row_stage(const uint4* st, const uint4* vs, int chunks, int lane,
                                                float (&acc)[4]) {
    if (chunks == kChainSegChunks) {
#pragma unroll
        for (int c = 0; c < kChainCL; ++c)
            fma_chunk<MODE>(st[c * 32], vs[(c * 2) * 32], vs[(c * 2 + 1) * 32], acc);
    } else {
#pragma unroll 1
        for (int c = 0; c < kChainCL; ++c)
            if (c * 32 + lane < chunks)
                fma_chunk<MODE>(st[c * 32], vs[(c * 2) * 32], vs[(c * 2 + 1) * 32], acc);
    }
}

// done[0] is the CTA ticket of the launch, done[1 + i] the number of CTAs that
// have finished op i.  All are zero between launches (the last CTA resets them).
// EARLY: the caller promises that nothing in flight writes the matrices or the
// table, so the producer starts before the stream-order wait.
template <bool EARLY>
__global__ void __launch_bounds__(kChainThreads, 1)
gemv_chain_kernel(const ChainOp* __restrict__ ops, int n_ops, unsigned int* __restrict__ done,
                  unsigned int* __restrict__ status, const __grid_constant__ ChainArArgs ar) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(128) unsigned char smem[];
    uint4* vec = reinterpret_cast<uint4*>(smem);                    // two buffers of kChainTile / 8 uint4
    unsigned char* ring = smem + 2 * kChainVecBytes;
    const uint32_t ring_s = smem_u32(ring);
    unsigned char* bar_mem = ring + kChainStages * kChainStageBytes;
    const uint32_t bars = smem_u32(bar_mem);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kChainStages + s); };
    auto vec_full = [&](int b) { return bars + 8u * (2 * kChainStages + b); };
    auto vec_empty = [&](int b) { return bars + 8u * (2 * kChainStages + 2 + b); };
    unsigned int* op_cnt = reinterpret_cast<unsigned int*>(bar_mem + 8 * kChainBarriers);
    uint4* table_w = reinterpret_cast<uint4*>(bar_mem + 8 * kChainBarriers + 8 * 4);
    const uint4* table = table_w;
    float* ar_stage = reinterpret_cast<float*>(table_w + 3 * kChainCachedOps);          // [slot][row of the task]
    unsigned int* ar_cnt = reinterpret_cast<unsigned int*>(ar_stage + kChainArSlots * kChainCW);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kChainStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), kChainCW);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(vec_full(b), 1);
            mbar_init(vec_empty(b), kChainCW);
        }
        for (int i = 0; i < 8; ++i) op_cnt[i] = 0u;
        for (int i = 0; i < kChainArSlots; ++i) ar_cnt[i] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (!EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");
    // Every warp walks the table.  A CTA that holds no rows of an op passes it in far less
    // time than a load from L2 takes under a full HBM stream (measured: 0.3 us per op when
    // the entries came from global memory one op ahead), so the table is copied to shared
    // memory once.  (EARLY: the caller has promised that nothing in flight writes it.)
    for (int i = threadIdx.x; i < 3 * min(n_ops, kChainCachedOps); i += kChainThreads)
        table_w[i] = __ldg(reinterpret_cast<const uint4*>(ops) + i);
    __syncthreads();

    if (warp == kChainCW + 2) {
        // ---------------------------------------------------- reduce warp --
        if (ar.world > 0) {
            if (EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");
            // this call's number: one more than the calls completed on this rank
            unsigned int epoch = __ldcg(ar.flags[ar.rank] + kArEpochWord) + 1u;
            if (epoch == 0u) epoch = 2u;   // 0 is the tag of an untouched inbox; keep the parity
            bool alive = true;
            ChainOp next = chain_load_op(ops, table, 0, n_ops);
            for (int op = 0; op < n_ops && alive; ++op) {
                const ChainOp d = next;
                next = chain_load_op(ops, table, op + 1, n_ops);
                const int ai = d.ar_index();
                if (ai < 0) continue;
                const ChainGeom g = chain_geom(d);
                for (int r0 = g.row_begin; r0 < g.row_end && alive; r0 += 32) {
                    const int row = r0 + lane;
                    if (row < g.row_end) {
                        // The ranks' pairs for this row, eight ranks at a time with all eight loads
                        // in flight (asked for one after the other, every rank costs an L2 round
                        // trip, and 44 all-reduced ops x 8 ranks of those were most of an 8-GPU
                        // token); a pair whose tag is not this call's yet is polled on its own.
                        float total = 0.f;
                        for (int q0 = 0; q0 < ar.world && alive; q0 += 8) {
                            uint2 x[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if (q0 + i < ar.world)
                                    x[i] = ld_volatile_v2(ar.inbox[ar.rank] + 2 * ar.pair_index(epoch, ai, q0 + i, row));
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                if (q0 + i < ar.world) {
                                    if (x[i].y != epoch) {
                                        const float* src = ar.inbox[ar.rank] + 2 * ar.pair_index(epoch, ai, q0 + i, row);
                                        const unsigned long long t0 = global_timer_ns();
                                        do {
                                            x[i] = ld_volatile_v2(src);
                                            if (global_timer_ns() - t0 > kWaitLimitNs) {
                                                atomicOr(status, 2u);   // that rank's sums did not arrive in time
                                                alive = false;
                                                break;
                                            }
                                        } while (x[i].y != epoch);
                                    }
                                    // rank order: the same bits everywhere
                                    total = q0 + i == 0 ? __uint_as_float(x[i].x) : total + __uint_as_float(x[i].x);
                                }
                            }
                        }
                        if (alive && bounds_ok(row < d.M)) chain_store_row(d, row, total);
                    }
                    alive = __all_sync(0xFFFFFFFFu, alive);
                }
                if (alive && d.signal() && g.row_end > g.row_begin) {
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicAdd(done + 1 + op, 1u);
                }
            }
        }
    } else if (warp == kChainCW) {
        // ------------------------------------------------------- producer --
        int s = 0;
        uint32_t round = 0;
        bool alive = true;
        ChainOp next = chain_load_op(ops, table, 0, n_ops);
        for (int op = 0; op < n_ops && alive; ++op) {
            const ChainOp d = next;
            next = chain_load_op(ops, table, op + 1, n_ops);
            const ChainGeom g = chain_geom(d);
            const size_t row_bytes = (size_t)d.N;
            for (int task = 0; task < g.n_tasks && alive; ++task) {
                const int row0 = g.row_begin + task * kChainCW;
                const int rows = min(kChainCW, g.row_end - row0);
                for (int seg = 0; seg < g.n_seg; ++seg) {
                    if (round > 0 && !mbar_wait_backoff(empty_bar(s), (round & 1u) ^ 1u, status, 20)) {
                        alive = false;
                        break;
                    }
                    const int chunks = min(kChainSegChunks, g.n16 - seg * kChainSegChunks);
                    const uint32_t bytes = (uint32_t)chunks * 16u;
                    if (lane == 0) mbar_arrive_expect_tx(full_bar(s), bytes * (uint32_t)rows);
                    if (g.n_seg == 1) {
                        // The rows of a task lie back to back in memory when a row is one segment,
                        // and the stage keeps them back to back too (row stride = row length).
                        // The copy engine takes ~50-70 ns per request whatever its size (16 requests
                        // of 2 KiB cap an SM at ~29 KB/us, below its share of HBM), so the task goes
                        // as at most four requests of four rows each instead of one per row.
                        const int r_first = lane * 4, r_count = min(4, rows - r_first);
                        if (lane < 4 && r_count > 0 && bounds_ok(row0 + r_first + r_count <= d.M))
                            bulk_load(ring_s + s * kChainStageBytes + (uint32_t)r_first * bytes,
                                      d.m + (size_t)(row0 + r_first) * row_bytes, (uint32_t)r_count * bytes,
                                      full_bar(s));
                    } else if (lane < rows &&
                               bounds_ok(row0 + lane < d.M && (size_t)seg * kChainSegBytes + bytes <= row_bytes)) {
                        bulk_load(ring_s + s * kChainStageBytes + lane * kChainSegBytes,
                                  d.m + (size_t)(row0 + lane) * row_bytes + (size_t)seg * kChainSegBytes,
                                  bytes, full_bar(s));
                    }
                    if (++s == kChainStages) { s = 0; ++round; }
                }
            }
        }
        if (!alive) {
            const unsigned long long t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 1000000ull) {}   // let the copies in flight land
        }
    } else if (warp == kChainCW + 1) {
        // ---------------------------------------------------- vector warp --
        if (EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");  // vectors and counters
        int vec_idx = -1;
        const uint32_t* staged_v = nullptr;
        int staged_n = -1, staged_mode = -1, staged_wait = -1;   // staged_wait: the op that vector was waited for
        bool alive = true;
        ChainOp next = chain_load_op(ops, table, 0, n_ops);
        for (int op = 0; op < n_ops && alive; ++op) {
            const ChainOp d = next;
            next = chain_load_op(ops, table, op + 1, n_ops);
            const ChainGeom g = chain_geom(d);
            if (g.n_tasks == 0) continue;
            if (d.v == staged_v && d.N == staged_n && d.mode() == staged_mode &&
                (d.wait_op < 0 || d.wait_op == staged_wait)) continue;
            staged_v = d.v; staged_n = d.N; staged_mode = d.mode(); staged_wait = d.wait_op;
            ++vec_idx;
            const int b = vec_idx & 1;
            if (vec_idx >= 2 && !mbar_wait_backoff(vec_empty(b), (uint32_t)((vec_idx >> 1) - 1) & 1u, status, 100)) break;
            if (d.wait_op >= 0) {
                // the vector is op wait_op's output: all CTAs that hold rows of it must be done
                const ChainOp w = chain_load_op(ops, table, d.wait_op, n_ops);
                const unsigned int target = (unsigned int)min((int)gridDim.x, (w.M + kChainCW - 1) / kChainCW);  // CTAs that hold rows of it
                const unsigned int* flag = done + 1 + d.wait_op;
                if (ld_acquire_gpu(flag) < target) {
                    const unsigned long long t0 = global_timer_ns();
                    while (ld_acquire_gpu(flag) < target) {
                        if (global_timer_ns() - t0 > kWaitLimitNs) {
                            atomicOr(status, 4u);   // an op this one depends on did not finish in time
                            alive = false;
                            break;
                        }
                    }
                }
                alive = __all_sync(0xFFFFFFFFu, alive);   // the lanes leave together
                if (!alive) break;
            }
            // chunk c (16 codes) -> uint4 (c / 32 * 2 + k) * 32 + c % 32, k = 0, 1: the FP16
            // pairs of its first and second eight codes (the layout fma_chunk reads)
            uint4* dst = vec + b * (kChainTile / 8);
            const uint4* src = reinterpret_cast<const uint4*>(d.v);
            const int fill = g.n_seg * kChainSegChunks;
            constexpr int kBatch = 8;
            for (int c0 = lane; c0 < fill; c0 += 32 * kBatch) {
                uint4 raw[kBatch];
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int c = c0 + 32 * u;
                    raw[u] = c < g.n16 ? ld_l2(src + c) : make_uint4(0, 0, 0, 0);  // past N: code 0 = +0.0
                }
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int c = c0 + 32 * u;
                    if (c < fill) {
                        uint4 lo, hi;
                        if (d.mode() == kE5M2) {
                            decode_word_h2<kE5M2>(raw[u].x, lo.x, lo.y);
                            decode_word_h2<kE5M2>(raw[u].y, lo.z, lo.w);
                            decode_word_h2<kE5M2>(raw[u].z, hi.x, hi.y);
                            decode_word_h2<kE5M2>(raw[u].w, hi.z, hi.w);
                        } else {
                            decode_word_h2<kE4M3>(raw[u].x, lo.x, lo.y);
                            decode_word_h2<kE4M3>(raw[u].y, lo.z, lo.w);
                            decode_word_h2<kE4M3>(raw[u].z, hi.x, hi.y);
                            decode_word_h2<kE4M3>(raw[u].w, hi.z, hi.w);
                        }
                        dst[((c >> 5) * 2) * 32 + (c & 31)] = lo;
                        dst[((c >> 5) * 2 + 1) * 32 + (c & 31)] = hi;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(vec_full(b));
        }
    } else {
        // ------------------------------------------------------ consumers --
        if (EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");  // before any output is written
        unsigned int epoch = 0;
        if (ar.world > 0) {
            epoch = __ldcg(ar.flags[ar.rank] + kArEpochWord) + 1u;
            if (epoch == 0u) epoch = 2u;
        }
        int s = 0;
        uint32_t phase = 0;
        int vec_idx = -1, sig_idx = 0, ar_seq = 0;
        const uint32_t* staged_v = nullptr;
        int staged_n = -1, staged_mode = -1, staged_wait = -1;   // staged_wait: the op that vector was waited for
        bool alive = true;
        const uint4* const ring_lane = reinterpret_cast<const uint4*>(ring) + lane;
        ChainOp next = chain_load_op(ops, table, 0, n_ops);
        for (int op = 0; op < n_ops && alive; ++op) {
            const ChainOp d = next;
            next = chain_load_op(ops, table, op + 1, n_ops);
            const ChainGeom g = chain_geom(d);
            if (g.n_tasks == 0) continue;
            if (!(d.v == staged_v && d.N == staged_n && d.mode() == staged_mode &&
                (d.wait_op < 0 || d.wait_op == staged_wait))) {
                staged_v = d.v; staged_n = d.N; staged_mode = d.mode(); staged_wait = d.wait_op;
                if (vec_idx >= 0) {   // done with the previous vector
                    __syncwarp();
                    if (lane == 0) mbar_arrive(vec_empty(vec_idx & 1));
                }
                ++vec_idx;
                if (!mbar_wait_backoff(vec_full(vec_idx & 1), (uint32_t)(vec_idx >> 1) & 1u, status)) break;
            }
            const uint4* vbase = vec + (vec_idx & 1) * (kChainTile / 8) + lane;
            for (int task = 0; task < g.n_tasks && alive; ++task) {
                // Row `slot` of the task belongs to warp (slot + shift) % 16, the shift moving
                // with op and task: a short task (14 of 16 rows, 2 rows of a 256-row matrix)
                // then idles different warps -- and different schedulers -- each time, and
                // because the warps run up to a ring's depth apart the load evens out.
                const int slot = (warp - (5 * op + 3 * task)) & (kChainCW - 1);
                const int row = g.row_begin + task * kChainCW + slot;
                const bool has_row = row < g.row_end;   // warp-uniform
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int seg = 0; seg < g.n_seg; ++seg) {
                    if (!mbar_wait_backoff(full_bar(s), phase, status)) {
                        alive = false;
                        break;
                    }
                    if (has_row) {
                        // a one-segment row sits at slot * (row length) in the stage, see the producer
                        const uint4* st = ring_lane + s * (kChainCW * kChainSegChunks) +
                                          slot * (g.n_seg == 1 ? g.n16 : kChainSegChunks);
                        const uint4* vs = vbase + (seg * kChainCL * 2) * 32;
                        const int chunks = min(kChainSegChunks, g.n16 - seg * kChainSegChunks);
                        if (d.mode() == kE5M2) chain_row_stage<kE5M2>(st, vs, chunks, lane, acc);
                        else chain_row_stage<kE4M3>(st, vs, chunks, lane, acc);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_bar(s));
                    if (++s == kChainStages) { s = 0; phase ^= 1u; }
                }
                if (!alive) break;
                if (has_row) {
                    float sums[1] = {(acc[0] + acc[1]) + (acc[2] + acc[3])};
                    warp_reduce_rows<1>(sums, lane);   // every lane holds the row's sum
                    const int ai = d.ar_index();
                    if (ai >= 0) {
                        // Partial sum of a column-sharded op.  The task's (up to) 16 sums meet in
                        // shared memory and the warp that brings the last one sends them to every
                        // rank (this one included) as (sum, call number) pairs, 128 contiguous bytes
                        // per rank in 16-byte stores: one NVLink packet per rank and task instead
                        // of one per rank and row, which is what the links charge for.  The reduce
                        // warps do the rest.
                        const int aslot = ar_seq & (kChainArSlots - 1);
                        const int row0 = g.row_begin + task * kChainCW;
                        const int t_rows = min(kChainCW, g.row_end - row0);
                        if (lane == 0) ar_stage[aslot * kChainCW + slot] = sums[0];
                        __threadfence_block();
                        unsigned int before = 0;
                        if (lane == 0) before = atomicAdd(ar_cnt + aslot, 1u);
                        before = __shfl_sync(0xFFFFFFFFu, before, 0);
                        if (before == (unsigned int)t_rows - 1u) {
                            if (lane == 0) ar_cnt[aslot] = 0u;
                            __threadfence_block();
                            const int j = lane & 7;                       // rows 2j, 2j + 1 of the task
                            const float s0 = 2 * j < t_rows ? ar_stage[aslot * kChainCW + 2 * j] : 0.f;
                            const float s1 = 2 * j + 1 < t_rows ? ar_stage[aslot * kChainCW + 2 * j + 1] : 0.f;
                            for (int q0 = 0; q0 < ar.world; q0 += 4) {
                                const int q = q0 + (lane >> 3);
                                if (q < ar.world && 2 * j < t_rows)
                                    st_volatile_v4(ar.inbox[q] + 2 * ar.pair_index(epoch, ai, ar.rank, row0 + 2 * j),
                                                   make_uint4(__float_as_uint(s0), epoch, __float_as_uint(s1), epoch));
                            }
                        }
                    } else if (lane == 0 && bounds_ok(row >= 0 && row < d.M)) {
                        chain_store_row(d, row, sums[0]);
                    }
                }
                ++ar_seq;   // every warp counts every task: the shared-memory slot of a task's partial sums
            }
            if (!alive) break;
            if (d.signal() && d.ar_index() < 0) {   // all-reduced ops are signalled by the reduce warp
                // This warp's rows of the op are written.  The warps count themselves in with a
                // release at CTA scope; the last one, having seen them all, issues the one
                // GPU-scope fence (which thereby covers every warp's rows) and counts the CTA
                // in done[op].
                __threadfence_block();
                __syncwarp();
                if (lane == 0) {
                    unsigned int* cnt = op_cnt + (sig_idx & 7);
                    if (atomicAdd(cnt, 1u) == kChainCW - 1) {
                        *cnt = 0u;
                        __threadfence();
                        atomicAdd(done + 1 + op, 1u);
                    }
                }
            }
            ++sig_idx;
        }
    }
    // ---- every role ends here: the last CTA of the launch zeroes the counters ----
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            for (int i = 0; i <= n_ops; ++i) done[i] = 0u;
            if (ar.world > 0) {   // the call is complete on this rank: count it
                unsigned int* my_flags = ar.flags[ar.rank];
                unsigned int epoch = my_flags[kArEpochWord] + 1u;
                if (epoch == 0u) epoch = 2u;
                my_flags[kArEpochWord] = epoch;
            }
        }
    }
}

}  // namespace feather
