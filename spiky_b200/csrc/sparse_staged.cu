// Table-ownership ("staged") kernels of the sparse non-sequence layer.
//
// With a batch of a few hundred samples nearly every row of a 256-row table is selected by some sample, so the
// whole table has to come from HBM anyway; the gather kernels (nonseq_sparse.cu) fetch it as random 64-100 byte row
// reads and are bound by the request rate.  Here a thread block instead OWNS a contiguous range of detectors for a
// tile of 512 samples: a producer warp streams the detectors' tables, one after the other, into a ring of
// shared-memory slots with bulk asynchronous copies (cp.async.bulk, completion counted on an mbarrier; plain
// single-CTA copies of this GPU's own memory), and 16 consumer warps (32 samples each) pick their samples' rows out
// of shared memory.  HBM sees one sequential read of the tables; the random accesses hit shared memory.
//
//   forward          the lanes of a group read one sample's row side by side and keep the running sums of (sample,
//                    synapse) over the detectors of a chunk in registers; one reduction per (sample, chunk part,
//                    target) goes to y when the chunk ends
//   input gradient   lane L reads the selected and the alternative row of sample L, forms
//                    sum_p dY[target(p)] * (W[row + p] - W[alt + p]) and makes the sample's two dX updates
//
// The detectors of the layer (times the sample tiles) are split evenly over one block per SM; a block walks its
// range chunk by chunk.  Every wait on an mbarrier is bounded (kWaitLimitCycles): a wait that runs out counts an error
// in g_wait_errors (lutb_device_wait_errors), raises the block's abort flag, and the block leaves after a bounded
// wait for its own copies in flight.
#include "sparse_staged.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "mbarrier.cuh"
#include "sparse_view.cuh"

namespace lutb {

constexpr int kConsumerWarps = 16;
constexpr int kStagedThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileSamples = kConsumerWarps * 32;
constexpr int kChunkSlots = 32;     // detector slots per chunk in the linear work order
constexpr int kMaxStages = 8;
constexpr int kMinStages = 3;
constexpr int kFwdTile = 4;         // detectors whose table indices a lane holds at a time (forward)
constexpr int kDxTile = 2;          // same for the input gradient (it also holds min_k and min_delta)

__device__ int g_wait_errors = 0;

struct StagedArgs {
    SparseView sp;
    const float *W;
    int64_t n_weights;
    int64_t batch;
    int64_t slots_per_tile;   // n_chunks * kChunkSlots
    int64_t total_slots;      // slots_per_tile * number of sample tiles
    int n_outputs, n_detectors, n_inputs, n_anchors;
    int slot_floats;
    int n_stages;
    int forward;   // 1: forward kernel, 0: input gradient (the two weigh tables differently when splitting the work)
};

// ------------------------------------------------------------------------------------------ work order
// Linear order of the work: sample tile major, then chunk, then detector slot (kChunkSlots per chunk; slots beyond a
// chunk's detector count are empty).  A block owns [lo, hi) of it and walks it in units: the part of one chunk that
// lies inside the range.
struct Unit {
    ChunkStatic cs;
    int d0, d1;        // detectors [d0, d1) of the chunk, already clipped to its detector count
    int64_t b0;        // first sample of the tile
    int64_t next_pos;  // position behind this unit
};

__device__ __forceinline__ Unit decode_unit(const StagedArgs &a, int64_t pos, int64_t hi) {
    Unit u;
    const int64_t bt = pos / a.slots_per_tile;
    const int64_t r = pos - bt * a.slots_per_tile;
    const int64_t c = r / kChunkSlots;
    const int s0 = (int)(r - c * kChunkSlots);
    const int s1 = (int)min((int64_t)kChunkSlots, s0 + (hi - pos));
    u.cs = load_chunk(a.sp, c);
    u.d0 = min(s0, u.cs.ndet);
    u.d1 = min(s1, u.cs.ndet);
    u.b0 = bt * kTileSamples;
    u.next_pos = pos + (s1 - s0);
    return u;
}

// Rows can be read with 64-bit loads when every row starts at an even slot and no hole lies inside a row.
__device__ __forceinline__ bool rows_vectorisable(const StagedArgs &a, const ChunkStatic &cs) {
    return (cs.stride & 1) == 0 && hole_offset(cs.P - 1, a.sp) == 0;
}

// Relative cost of one table of a chunk for the consumers (measured on B200: a fixed part for the hand-over of the
// slot, then the row reads).  Forward: one row read per sample-group of the warp (32 / 16 / 8 per table).  Input
// gradient: every lane reads its own two rows; rows that need one 32-bit load per synapse cost about three times the
// 64-bit ones.
__device__ __forceinline__ int table_cost(const StagedArgs &a, const ChunkStatic &cs) {
    if (a.forward) return 8 + (cs.P <= 8 ? 8 : cs.P <= 16 ? 16 : 32);
    const int nj = cs.P <= 8 ? 8 : cs.P <= 16 ? 16 : cs.P <= 20 ? 20 : cs.P <= 28 ? 28 : 32;
    return rows_vectorisable(a, cs) ? 8 + nj : 8 + 3 * (cs.P <= 8 ? 8 : cs.P <= 16 ? 16 : 32);
}

constexpr int kMaxBalanced = 2 * kStagedThreads;   // chunk instances the cost-balanced split can look at

// [lo, hi) of the block in the linear work order.  The tables are split by COST, not by count: the block with the
// slow tables would otherwise set the kernel's time.  Every block looks at all chunks (a few hundred 32-byte
// records), sums their cost and finds the two positions where the running cost crosses its share's borders;
// neighbouring blocks evaluate the same border the same way, so the ranges tile the work exactly.  Layers with more
// chunk instances than kMaxBalanced fall back to an even split by count.
__device__ void block_range(const StagedArgs &a, int64_t *lo, int64_t *hi) {
    __shared__ int32_t s_cost[kMaxBalanced];
    __shared__ long long s_border[2];
    const int64_t n_items = a.total_slots / kChunkSlots;   // chunk instances (chunks x sample tiles)
    if (n_items > kMaxBalanced) {
        const int64_t per = (a.total_slots + gridDim.x - 1) / gridDim.x;
        *lo = min(a.total_slots, (int64_t)blockIdx.x * per);
        *hi = min(a.total_slots, *lo + per);
        return;
    }
    for (int64_t i = threadIdx.x; i < n_items; i += blockDim.x) {
        const ChunkStatic cs = load_chunk(a.sp, i % a.sp.n_chunks);
        s_cost[i] = cs.ndet * table_cost(a, cs);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        long long total = 0;
        for (int64_t i = lane; i < n_items; i += 32) total += s_cost[i];
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) total += __shfl_xor_sync(0xffffffffu, total, m);
        const long long t_lo = total * blockIdx.x / gridDim.x, t_hi = total * (blockIdx.x + 1) / gridDim.x;
        if (lane == 0) { s_border[0] = a.total_slots; s_border[1] = a.total_slots; }
        __syncwarp();
        long long run = 0;   // cost of all items before this group of 32
        for (int64_t base = 0; base < n_items; base += 32) {
            const int64_t i = base + lane;
            const long long c = i < n_items ? s_cost[i] : 0;
            long long incl = c;
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const long long up = __shfl_up_sync(0xffffffffu, incl, m);
                if (lane >= m) incl += up;
            }
            const long long excl = run + incl - c;
            if (c > 0) {
                const ChunkStatic cs = load_chunk(a.sp, i % a.sp.n_chunks);
                const int w = (int)(c / cs.ndet);
                // the border lies inside this item: so many whole tables of it belong to the earlier block
                if (t_lo >= excl && t_lo < excl + c) s_border[0] = i * kChunkSlots + (t_lo - excl) / w;
                if (t_hi >= excl && t_hi < excl + c) s_border[1] = i * kChunkSlots + (t_hi - excl) / w;
            }
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();
    *lo = s_border[0];
    *hi = s_border[1];
}

struct RingPos {
    uint32_t slot, phase;
    __device__ __forceinline__ void advance(int n_stages) {
        if (++slot == (uint32_t)n_stages) { slot = 0; phase ^= 1u; }
    }
};

struct Ring {
    float *base;
    uint32_t full0, empty0;   // shared-window addresses of the first "table arrived" / "slot released" barrier
    volatile int *abort_flag;
};

__device__ __forceinline__ void report_wait_error(const Ring &ring) {
    atomicAdd(&g_wait_errors, 1);
    *ring.abort_flag = 1;
}

// Producer warp: streams the tables of the block's range into the ring.
__device__ void producer_loop(const StagedArgs &a, const Ring &ring, int64_t lo, int64_t hi, int lane) {
    RingPos rp{0u, 0u};
    uint32_t issued = 0;
    bool ok = true;
    for (int64_t pos = lo; pos < hi && ok;) {
        const Unit u = decode_unit(a, pos, hi);
        pos = u.next_pos;
        for (int d = u.d0; d < u.d1; d++) {
            // a fresh barrier passes the wait for parity 1, so the first round does not wait
            if (!mbar_wait(ring.empty0 + 8 * rp.slot, rp.phase ^ 1u) || *ring.abort_flag) { ok = false; break; }
            if (lane == 0) {
                const int64_t src0 = u.cs.wbase0 + (int64_t)d * u.cs.table;
                // the last row's trailing hole lies behind the end of the weight array: never read it
                const int64_t avail = min((int64_t)u.cs.table, a.n_weights - src0);
                const uint32_t bulk = (uint32_t)(avail * 4) & ~15u;
                float *dst = ring.base + (size_t)rp.slot * a.slot_floats;
                for (int64_t k = bulk / 4; k < avail; k++) dst[k] = __ldg(a.W + src0 + k);
                mbar_arrive_expect_tx(ring.full0 + 8 * rp.slot, bulk);
                if (bulk) bulk_copy_g2s(smem_u32(dst), a.W + src0, bulk, ring.full0 + 8 * rp.slot);
            }
            __syncwarp();
            rp.advance(a.n_stages);
            issued++;
        }
    }
    if (!ok) {
        if (lane == 0) report_wait_error(ring);
        // the block is leaving early: give the copies still in flight a bounded time to land
        const uint32_t n = min(issued, (uint32_t)a.n_stages);
        for (uint32_t k = 0; k < n; k++) {
            const uint32_t item = issued - 1 - k;
            if (!mbar_wait(ring.full0 + 8 * (item % a.n_stages), (item / a.n_stages) & 1u)) break;
        }
    }
}

// Table indices of up to TILE detectors for the lane's own sample (zero where there is none).
template <int TILE>
__device__ __forceinline__ void load_tile_i32(const int32_t *__restrict__ src, int64_t b, int64_t batch, int n_detectors,
                                              int det, int n, int32_t (&out)[TILE]) {
#pragma unroll
    for (int k = 0; k < TILE; k++) out[k] = 0;
    if (b >= batch || n <= 0) return;
    const int32_t *p = src + b * (int64_t)n_detectors + det;
    if (TILE % 4 == 0 && n == TILE && ((n_detectors | det) & 3) == 0) {
#pragma unroll
        for (int k = 0; k + 3 < TILE; k += 4) {
            const int4 v = __ldg(reinterpret_cast<const int4 *>(p + k));
            out[k] = v.x; out[k + 1] = v.y; out[k + 2] = v.z; out[k + 3] = v.w;
        }
    } else if (TILE == 2 && n == TILE && ((n_detectors | det) & 1) == 0) {
        const int2 v = __ldg(reinterpret_cast<const int2 *>(p));
        out[0] = v.x; out[TILE - 1] = v.y;
    } else {
#pragma unroll
        for (int k = 0; k < TILE; k++)
            if (k < n) out[k] = __ldg(p + k);
    }
}

// First non-empty unit at or behind pos; false when the range holds none.
__device__ __forceinline__ bool next_unit(const StagedArgs &a, int64_t pos, int64_t hi, Unit &u) {
    while (pos < hi) {
        u = decode_unit(a, pos, hi);
        if (u.d1 > u.d0) return true;
        pos = u.next_pos;
    }
    return false;
}

// ------------------------------------------------------------------------------------------ forward
// Inside a consumer warp lane L works on sample L of the warp's 32 samples: it holds the sample's table indices and
// reads the sample's row of every table itself, all synapses of the row into registers (64-bit shared loads when
// rows start at even slots and have no holes inside, else one load per synapse).  No lane depends on another, so a
// table costs a warp a handful of independent loads and adds; the price is bank conflicts between the 32 random
// rows, which leaves shared memory about as busy as the copies that fill it.
// NJ: synapses per row rounded up to a multiple of 4; values beyond the row's real length are loaded and ignored.
// Synapses [J0, J0 + 4) of the row at `off` (64-bit loads need J0 even, which multiples of 4 are).
template <int J0, bool VEC>
__device__ __forceinline__ void load_row4(const float *slot, uint32_t off, const SparseView &sp, float (&w)[4]) {
    if constexpr (VEC) {
        const float2 v0 = *reinterpret_cast<const float2 *>(slot + off + J0);
        const float2 v1 = *reinterpret_cast<const float2 *>(slot + off + J0 + 2);
        w[0] = v0.x; w[1] = v0.y; w[2] = v1.x; w[3] = v1.y;
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++) w[j] = slot[off + J0 + j + hole_offset(J0 + j, sp)];
    }
}

// Keeps the compiler from hoisting the next group of row loads above the arithmetic of the current one (the
// registers of a 32-synapse row, twice for the input gradient, do not fit beside the running sums).
__device__ __forceinline__ void schedule_fence() { asm volatile("" ::: "memory"); }

template <int J0, int NJ, bool VEC>
__device__ __forceinline__ void add_row(const float *slot, uint32_t off, const SparseView &sp, float (&acc)[NJ]) {
    if constexpr (J0 < NJ) {
        float w[4];
        load_row4<J0, VEC>(slot, off, sp, w);
#pragma unroll
        for (int j = 0; j < 4; j++) acc[J0 + j] += w[j];
        if constexpr (J0 % 8 == 4) schedule_fence();
        add_row<J0 + 4, NJ, VEC>(slot, off, sp, acc);
    }
}

template <int J0, int NJ, bool VEC>
__device__ __forceinline__ float dot_row_difference(const float *slot, uint32_t off, uint32_t alt, const SparseView &sp,
                                                    const float (&gp)[NJ], int P, float g) {
    if constexpr (J0 < NJ) {
        float wr[4], wa[4];
        load_row4<J0, VEC>(slot, off, sp, wr);
        load_row4<J0, VEC>(slot, alt, sp, wa);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // slots beyond the row's length hold unrelated bits: keep them out of the sum
            const float d = J0 + j < P ? wr[j] - wa[j] : 0.f;
            g = fmaf(gp[J0 + j], d, g);
        }
        if constexpr (J0 % 8 == 4) schedule_fence();
        return dot_row_difference<J0 + 4, NJ, VEC>(slot, off, alt, sp, gp, P, g);
    } else {
        return g;
    }
}

// Forward, lane layout inside a consumer warp: LG lanes per sample (LG = 8, 16 or 32 >= synapses per row), 32 / LG
// samples side by side; lane (h, j) works on synapse j of the samples h * LG + i, i = 0 .. LG - 1, of the warp's 32
// samples, so a row is read by neighbouring lanes as one contiguous piece of shared memory (no bank conflicts inside
// a row) and the sums of a sample leave the warp as one reduction over neighbouring output cells.  Lane L also holds
// the table indices of sample L (its "own" sample), which the others fetch by shuffle.
template <int LG>
__device__ __forceinline__ bool forward_unit(const StagedArgs &a, const Unit &u, const Unit &nx, bool has_next,
                                             const Ring &ring, RingPos &rp, const int32_t *__restrict__ idx,
                                             int32_t (&raw)[kFwdTile], int warp, int lane, float *__restrict__ y) {
    const int h = lane / LG, j = lane - h * LG;
    const bool valid = j < u.cs.P;
    const int64_t bw = u.b0 + warp * 32;
    const bool warp_active = bw < a.batch;
    const int q = j + hole_offset(j, a.sp);
    float acc[LG];
#pragma unroll
    for (int i = 0; i < LG; i++) acc[i] = 0.f;
    for (int t0 = u.d0; t0 < u.d1; t0 += kFwdTile) {
        uint32_t ro[kFwdTile];
#pragma unroll
        for (int k = 0; k < kFwdTile; k++) ro[k] = (uint32_t)raw[k] * (uint32_t)u.cs.stride;
        // the indices of the next tile (of this unit or of the next one) travel while this tile is worked on
        if (t0 + kFwdTile < u.d1)
            load_tile_i32<kFwdTile>(idx, bw + lane, a.batch, a.n_detectors, u.cs.det0 + t0 + kFwdTile,
                                    min(kFwdTile, u.d1 - t0 - kFwdTile), raw);
        else if (has_next)
            load_tile_i32<kFwdTile>(idx, nx.b0 + warp * 32 + lane, a.batch, a.n_detectors, nx.cs.det0 + nx.d0,
                                    min(kFwdTile, nx.d1 - nx.d0), raw);
#pragma unroll
        for (int dd = 0; dd < kFwdTile; dd++) {
            if (t0 + dd < u.d1) {
                if (!mbar_wait(ring.full0 + 8 * rp.slot, rp.phase) || *ring.abort_flag) return false;
                if (warp_active) {
                    const float *tab = ring.base + (size_t)rp.slot * a.slot_floats + q;
                    // in batches of 8 rows: all row offsets first, then all row reads, then the additions, so that
                    // the shuffles and the shared-memory reads of a batch are in flight together instead of forming
                    // one dependent chain per row
                    constexpr int BATCH = 8;
#pragma unroll
                    for (int i0 = 0; i0 < LG; i0 += BATCH) {
                        uint32_t off[BATCH];
                        float val[BATCH];
#pragma unroll
                        for (int i = 0; i < BATCH; i++) off[i] = __shfl_sync(0xffffffffu, ro[dd], h * LG + i0 + i);
#pragma unroll
                        for (int i = 0; i < BATCH; i++) val[i] = valid ? tab[off[i]] : 0.f;
#pragma unroll
                        for (int i = 0; i < BATCH; i++) acc[i0 + i] += val[i];
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(ring.empty0 + 8 * rp.slot);
                rp.advance(a.n_stages);
            }
        }
    }
    if (warp_active && valid) {
        const int target = __ldg(a.sp.syn_target + u.cs.toff + j);
#pragma unroll
        for (int i = 0; i < LG; i++) {
            const int64_t b = bw + h * LG + i;
            if (b < a.batch) atomicAdd(y + b * a.n_outputs + target, acc[i]);
        }
    }
    return true;
}

// Shared memory: the ring, then the barriers (two per stage) and the abort flag.
__device__ __forceinline__ Ring setup_ring(const StagedArgs &a, unsigned char *smem) {
    Ring ring;
    ring.base = reinterpret_cast<float *>(smem);
    unsigned char *tail = smem + (size_t)a.n_stages * a.slot_floats * sizeof(float);
    ring.full0 = smem_u32(tail);
    ring.empty0 = ring.full0 + 8 * kMaxStages;
    ring.abort_flag = reinterpret_cast<volatile int *>(tail + 16 * kMaxStages);
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.n_stages; s++) {
            mbar_init(ring.full0 + 8 * s, 1);                 // the producer's arrive + the copy's bytes
            mbar_init(ring.empty0 + 8 * s, kConsumerWarps);   // one arrive per consumer warp
        }
        *ring.abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    return ring;
}

__global__ void __launch_bounds__(kStagedThreads, 1) sparse_forward_staged_kernel(StagedArgs a,
                                                                                const int32_t *__restrict__ idx,
                                                                                float *__restrict__ y) {
    extern __shared__ __align__(128) unsigned char smem[];
    const Ring ring = setup_ring(a, smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int64_t lo, hi;
    block_range(a, &lo, &hi);   // all threads: it synchronises the block
    if (warp == kConsumerWarps) {
        producer_loop(a, ring, lo, hi, lane);
        return;
    }
    Unit cur, nxt;
    bool has_cur = next_unit(a, lo, hi, cur);
    RingPos rp{0u, 0u};
    int32_t raw[kFwdTile];
    if (has_cur)
        load_tile_i32<kFwdTile>(idx, cur.b0 + warp * 32 + lane, a.batch, a.n_detectors, cur.cs.det0 + cur.d0,
                                min(kFwdTile, cur.d1 - cur.d0), raw);
    while (has_cur) {
        const bool has_next = next_unit(a, cur.next_pos, hi, nxt);
        bool ok;
#define LUTB_FWD_UNIT(LGV) forward_unit<LGV>(a, cur, nxt, has_next, ring, rp, idx, raw, warp, lane, y)
        if (cur.cs.P <= 8) ok = LUTB_FWD_UNIT(8);
        else if (cur.cs.P <= 16) ok = LUTB_FWD_UNIT(16);
        else ok = LUTB_FWD_UNIT(32);
#undef LUTB_FWD_UNIT
        if (!ok) {
            if (lane == 0) report_wait_error(ring);
            return;
        }
        cur = nxt;
        has_cur = has_next;
    }
}

// ------------------------------------------------------------------------------------------ input gradient
// Same mapping: lane L forms g = sum_p dY[target(p)] * (W[row + p] - W[alt + p]) of its own sample from its own two
// row reads (fp32, <= 32 terms), scales it by up() in double and makes the sample's two dX updates.
template <int NJ, bool VEC>
__device__ __forceinline__ bool input_grad_unit(const StagedArgs &a, const Unit &u, const Unit &nx, bool has_next,
                                                const Ring &ring, RingPos &rp, const int32_t *__restrict__ idx,
                                                const int32_t *__restrict__ min_k, const float *__restrict__ min_delta,
                                                const float *__restrict__ dY, const int2 *__restrict__ anchors,
                                                int32_t (&raw_i)[kDxTile], int32_t (&raw_k)[kDxTile],
                                                int32_t (&raw_m)[kDxTile], int warp, int lane, float *__restrict__ dX) {
    const int64_t bw = u.b0 + warp * 32;
    const bool warp_active = bw < a.batch;
    const int64_t own_b = bw + lane;
    const bool has_b = own_b < a.batch;
    // output gradients of the sample at the chunk's targets: the same for every detector of the chunk
    float gp[NJ];
    {
        const int32_t *tg = a.sp.syn_target + u.cs.toff;
        const float *dyb = dY + (has_b ? own_b : 0) * a.n_outputs;
#pragma unroll
        for (int j = 0; j < NJ; j++) gp[j] = (has_b && j < u.cs.P) ? __ldg(dyb + __ldg(tg + j)) : 0.f;
    }
    for (int t0 = u.d0; t0 < u.d1; t0 += kDxTile) {
        uint32_t ro[kDxTile], ao[kDxTile];
        int32_t ck[kDxTile];
        float cm[kDxTile];
#pragma unroll
        for (int k = 0; k < kDxTile; k++) {
            const uint32_t li = (uint32_t)raw_i[k];
            ro[k] = li * (uint32_t)u.cs.stride;
            ao[k] = (li ^ (1u << raw_k[k])) * (uint32_t)u.cs.stride;   // minimum-margin bit flipped
            ck[k] = raw_k[k];
            cm[k] = __int_as_float(raw_m[k]);
        }
        {
            int64_t pb;
            int pdet, pn;
            if (t0 + kDxTile < u.d1) { pb = own_b; pdet = u.cs.det0 + t0 + kDxTile; pn = min(kDxTile, u.d1 - t0 - kDxTile); }
            else if (has_next) { pb = nx.b0 + warp * 32 + lane; pdet = nx.cs.det0 + nx.d0; pn = min(kDxTile, nx.d1 - nx.d0); }
            else { pb = 0; pdet = 0; pn = 0; }
            load_tile_i32<kDxTile>(idx, pb, a.batch, a.n_detectors, pdet, pn, raw_i);
            load_tile_i32<kDxTile>(min_k, pb, a.batch, a.n_detectors, pdet, pn, raw_k);
            load_tile_i32<kDxTile>(reinterpret_cast<const int32_t *>(min_delta), pb, a.batch, a.n_detectors, pdet, pn, raw_m);
        }
#pragma unroll
        for (int dd = 0; dd < kDxTile; dd++) {
            if (t0 + dd < u.d1) {
                if (!mbar_wait(ring.full0 + 8 * rp.slot, rp.phase) || *ring.abort_flag) return false;
                if (warp_active) {
                    const float *slot = ring.base + (size_t)rp.slot * a.slot_floats;
                    const float g = dot_row_difference<0, NJ, VEC>(slot, ro[dd], ao[dd], a.sp, gp, u.cs.P, 0.f);
                    if (has_b) {
                        const double du = surrogate_up(cm[dd]) * (double)g;
                        if (fabs(du) > kEps) {
                            const int2 an = __ldg(anchors + (size_t)(u.cs.det0 + t0 + dd) * a.n_anchors + ck[dd]);
                            float *dxb = dX + own_b * a.n_inputs;
                            atomicAdd(dxb + an.x, (float)du);
                            atomicAdd(dxb + an.y, -(float)du);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(ring.empty0 + 8 * rp.slot);
                rp.advance(a.n_stages);
            }
        }
    }
    return true;
}

__global__ void __launch_bounds__(kStagedThreads, 1) sparse_input_grad_staged_kernel(
    StagedArgs a, const int32_t *__restrict__ idx, const int32_t *__restrict__ min_k, const float *__restrict__ min_delta,
    const float *__restrict__ dY, const int2 *__restrict__ anchors, float *__restrict__ dX) {
    extern __shared__ __align__(128) unsigned char smem[];
    const Ring ring = setup_ring(a, smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int64_t lo, hi;
    block_range(a, &lo, &hi);   // all threads: it synchronises the block
    if (warp == kConsumerWarps) {
        producer_loop(a, ring, lo, hi, lane);
        return;
    }
    Unit cur, nxt;
    bool has_cur = next_unit(a, lo, hi, cur);
    RingPos rp{0u, 0u};
    int32_t raw_i[kDxTile], raw_k[kDxTile], raw_m[kDxTile];
    if (has_cur) {
        const int64_t b = cur.b0 + warp * 32 + lane;
        const int det = cur.cs.det0 + cur.d0, n = min(kDxTile, cur.d1 - cur.d0);
        load_tile_i32<kDxTile>(idx, b, a.batch, a.n_detectors, det, n, raw_i);
        load_tile_i32<kDxTile>(min_k, b, a.batch, a.n_detectors, det, n, raw_k);
        load_tile_i32<kDxTile>(reinterpret_cast<const int32_t *>(min_delta), b, a.batch, a.n_detectors, det, n, raw_m);
    }
    while (has_cur) {
        const bool has_next = next_unit(a, cur.next_pos, hi, nxt);
        bool ok;
#define LUTB_DX_UNIT(NJV, VECV) \
    input_grad_unit<NJV, VECV>(a, cur, nxt, has_next, ring, rp, idx, min_k, min_delta, dY, anchors, raw_i, raw_k, raw_m, warp, lane, dX)
        if (rows_vectorisable(a, cur.cs)) {
            if (cur.cs.P <= 8) ok = LUTB_DX_UNIT(8, true);
            else if (cur.cs.P <= 16) ok = LUTB_DX_UNIT(16, true);
            else if (cur.cs.P <= 20) ok = LUTB_DX_UNIT(20, true);
            else if (cur.cs.P <= 28) ok = LUTB_DX_UNIT(28, true);
            else ok = LUTB_DX_UNIT(32, true);
        } else {
            if (cur.cs.P <= 8) ok = LUTB_DX_UNIT(8, false);
            else if (cur.cs.P <= 16) ok = LUTB_DX_UNIT(16, false);
            else ok = LUTB_DX_UNIT(32, false);
        }
#undef LUTB_DX_UNIT
        if (!ok) {
            if (lane == 0) report_wait_error(ring);
            return;
        }
        cur = nxt;
        has_cur = has_next;
    }
}

// ------------------------------------------------------------------------------------------ host side
static size_t slot_bytes_of(const lutb_sparse_index *sp) { return (((size_t)sp->max_table_slots * 4) + 127) & ~(size_t)127; }

static int stages_of(const lutb_sparse_index *sp) {
    // barriers + abort flag behind the ring, and the kernels' static shared memory (cost table of block_range)
    const size_t tail = 16 * kMaxStages + 128 + (kMaxBalanced * sizeof(int32_t) + 256);
    const size_t slot = slot_bytes_of(sp);
    if (slot == 0 || slot + tail > (size_t)kMaxSmemPerBlock) return 0;
    const size_t n = ((size_t)kMaxSmemPerBlock - tail) / slot;
    return (int)(n > (size_t)kMaxStages ? kMaxStages : n);
}

bool sparse_staged_possible(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, const float *weights) {
    if (cfg->int_mode != 0 || cfg->seq_len != 1) return false;
    if (sp->max_count > 32 || sp->max_table_slots <= 0 || sp->max_table_slots > 65535 || !sp->tables_aligned16) return false;
    if ((reinterpret_cast<uintptr_t>(weights) & 15) != 0) return false;
    return stages_of(sp) >= kMinStages;
}

bool sparse_staged_preferred(int pass, const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch) {
    // whole tables are streamed whatever the batch: worth it once the batch selects most rows of a table anyway,
    // and when the layer has enough detectors to give every SM a range.  Input gradient: the staged kernel measured
    // slower than the gather kernel on B200 (both end up bound by the load/store unit: the two scattered dX
    // reductions per (sample, detector) cost the same in either, and 32 lanes reading 32 different rows of a table
    // in shared memory collide on its banks about as often as they would miss in L1), so it is never the
    // library's choice.
    if (pass != 0) return false;
    const int64_t rows = (int64_t)1 << cfg->n_anchors;
    return 2 * batch >= rows && cfg->n_detectors >= 4 * device_info().sm_count;
}

static int fill_args(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch, const float *weights,
                     bool forward, StagedArgs *a, unsigned *grid, size_t *smem) {
    a->forward = forward ? 1 : 0;
    a->sp = make_view(sp);
    a->W = weights;
    a->n_weights = sp->n_weights;
    a->batch = batch;
    a->slots_per_tile = sp->n_chunks * kChunkSlots;
    const int64_t tiles = (batch + kTileSamples - 1) / kTileSamples;
    a->total_slots = a->slots_per_tile * tiles;
    a->n_outputs = cfg->n_outputs; a->n_detectors = cfg->n_detectors; a->n_inputs = cfg->n_inputs;
    a->n_anchors = cfg->n_anchors;
    a->slot_floats = (int)(slot_bytes_of(sp) / 4);
    a->n_stages = stages_of(sp);
    LUTB_REQUIRE(a->n_stages >= kMinStages, LUTB_ERR_MODE, "detector tables too large for the shared-memory ring");
    const int sm = device_info().sm_count;
    // one block per SM; fewer when the layer is tiny (at least 8 detector slots per block)
    const int64_t want = (a->total_slots + 7) / 8;
    *grid = (unsigned)(want < sm ? want : sm);
    *smem = (size_t)a->n_stages * slot_bytes_of(sp) + 16 * kMaxStages + 128;
    return LUTB_OK;
}

template <typename K>
static int allow_smem(K kernel, size_t smem) {
    // per device, not cached across devices: the attribute is cheap to set
    LUTB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return LUTB_OK;
}

int launch_sparse_forward_staged(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                 const float *weights, const int32_t *idx, float *y, cudaStream_t stream) {
    StagedArgs a;
    unsigned grid;
    size_t smem;
    int rc = fill_args(cfg, sp, batch, weights, true, &a, &grid, &smem);
    if (rc) return rc;
    rc = allow_smem(sparse_forward_staged_kernel, smem);
    if (rc) return rc;
    KernelScope scope(K_SPARSE_FORWARD, stream);
    sparse_forward_staged_kernel<<<grid, kStagedThreads, smem, stream>>>(a, idx, y);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

int launch_sparse_input_grad_staged(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                    const float *weights, const float *dY, const int32_t *anchors, const int32_t *idx,
                                    const float *min_delta, const int32_t *min_k, float *dX, cudaStream_t stream) {
    StagedArgs a;
    unsigned grid;
    size_t smem;
    int rc = fill_args(cfg, sp, batch, weights, false, &a, &grid, &smem);
    if (rc) return rc;
    rc = allow_smem(sparse_input_grad_staged_kernel, smem);
    if (rc) return rc;
    KernelScope scope(K_SPARSE_INPUT_GRAD, stream);
    sparse_input_grad_staged_kernel<<<grid, kStagedThreads, smem, stream>>>(a, idx, min_k, min_delta, dY,
                                                                          reinterpret_cast<const int2 *>(anchors), dX);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

}  // namespace lutb

// Number of bounded device-side waits that ran out since the library was loaded on the current device (0 in a
// healthy run).  Synchronises the device.
extern "C" int lutb_device_wait_errors(int *count_out) {
    LUTB_REQUIRE(count_out != nullptr, LUTB_ERR_NULL, "count_out is NULL");
    LUTB_CUDA(cudaMemcpyFromSymbol(count_out, lutb::g_wait_errors, sizeof(int)));
    int peer = 0;
    const int rc = lutb::peer_wait_errors(&peer);
    if (rc) return rc;
    *count_out += peer;
    return LUTB_OK;
}
