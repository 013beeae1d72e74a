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
//   forward          each lane keeps the running sum of (its sample, its synapse) over the detectors of a chunk in
//                    a register; one reduction per (sample, chunk part, target) goes to y when the chunk ends
//   input gradient   per (sample, detector) the products dY[target(p)] * (W[row + p] - W[alt + p]) are summed over
//                    the lanes with a transpose-reduce, so that lane L ends with the sum of sample L and makes that
//                    sample's two dX updates itself
//
// The detectors of the layer (times the sample tiles) are split evenly over one block per SM; a block walks its
// range chunk by chunk.  Every wait on an mbarrier is bounded (kWaitLimitNs): a wait that runs out counts an error
// in g_wait_errors (lutb_device_wait_errors), raises the block's abort flag, and the block leaves after a bounded
// wait for its own copies in flight.
#include "sparse_staged.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "sparse_view.cuh"

namespace lutb {

constexpr int kConsumerWarps = 16;
constexpr int kStagedThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileSamples = kConsumerWarps * 32;
constexpr int kChunkSlots = 32;     // detector slots per chunk in the linear work order
constexpr int kMaxStages = 8;
constexpr int kMinStages = 3;
constexpr int kFwdTile = 8;         // detectors whose table indices a lane holds at a time (forward)
constexpr int kDxTile = 2;          // same for the input gradient (it also holds min_k)
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;

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
};

// ------------------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    while (!mbar_try_wait(bar, parity)) {
        if (global_timer_ns() - t0 > kWaitLimitNs) return false;
    }
    return true;
}
// One contiguous global -> shared copy; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

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

__device__ __forceinline__ void block_range(const StagedArgs &a, int64_t *lo, int64_t *hi) {
    const int64_t per = (a.total_slots + gridDim.x - 1) / gridDim.x;
    *lo = min(a.total_slots, (int64_t)blockIdx.x * per);
    *hi = min(a.total_slots, *lo + per);
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
__device__ void producer_loop(const StagedArgs &a, const Ring &ring, int lane) {
    int64_t lo, hi;
    block_range(a, &lo, &hi);
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
// Lane layout inside a consumer warp: LG lanes per sample (LG = 8, 16 or 32 >= synapses per row), 32 / LG samples
// side by side; lane (h, j) works on synapse j of the samples h * LG + i, i = 0 .. LG - 1, of the warp's 32 samples.
// Lane L also holds the table indices of sample L (its "own" sample), which the others fetch by shuffle.
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
#pragma unroll
                    for (int i = 0; i < LG; i++) {
                        const uint32_t off = __shfl_sync(0xffffffffu, ro[dd], h * LG + i);
                        if (valid) acc[i] += tab[off];
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
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
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
    if (warp == kConsumerWarps) {
        producer_loop(a, ring, lane);
        return;
    }
    int64_t lo, hi;
    block_range(a, &lo, &hi);
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
        if (cur.cs.P <= 8) ok = forward_unit<8>(a, cur, nxt, has_next, ring, rp, idx, raw, warp, lane, y);
        else if (cur.cs.P <= 16) ok = forward_unit<16>(a, cur, nxt, has_next, ring, rp, idx, raw, warp, lane, y);
        else ok = forward_unit<32>(a, cur, nxt, has_next, ring, rp, idx, raw, warp, lane, y);
        if (!ok) {
            if (lane == 0) report_wait_error(ring);
            return;
        }
        cur = nxt;
        has_cur = has_next;
    }
}

// ------------------------------------------------------------------------------------------ input gradient
// Same lane layout.  Per detector every lane forms its LG products, a butterfly of LG - 1 shuffles transposes and
// sums them so that lane (h, j) ends with the full sum of sample h * LG + j = its own sample, whose min_delta, min_k
// and table index it holds.  Partial sums are fp32 (<= 32 terms), the scaling by up() is done in double.
template <int LG>
__device__ __forceinline__ bool input_grad_unit(const StagedArgs &a, const Unit &u, const Unit &nx, bool has_next,
                                                const Ring &ring, RingPos &rp, const int32_t *__restrict__ idx,
                                                const int32_t *__restrict__ min_k, const float *__restrict__ min_delta,
                                                const float *__restrict__ dY, const int2 *__restrict__ anchors,
                                                int32_t (&raw_i)[kDxTile], int32_t (&raw_k)[kDxTile], int warp, int lane,
                                                float *__restrict__ dX) {
    const int h = lane / LG, j = lane - h * LG;
    const bool valid = j < u.cs.P;
    const int64_t bw = u.b0 + warp * 32;
    const bool warp_active = bw < a.batch;
    const int64_t own_b = bw + lane;
    const int q = j + hole_offset(j, a.sp);
    // output gradients of (sample, target(j)): the same for every detector of the chunk
    float gp[LG];
    {
        const int target = valid ? __ldg(a.sp.syn_target + u.cs.toff + j) : 0;
#pragma unroll
        for (int i = 0; i < LG; i++) {
            const int64_t b = bw + h * LG + i;
            gp[i] = (valid && b < a.batch) ? __ldg(dY + b * a.n_outputs + target) : 0.f;
        }
    }
    for (int t0 = u.d0; t0 < u.d1; t0 += kDxTile) {
        uint32_t pk[kDxTile];   // row offset | alternative row offset << 16
        int32_t ck[kDxTile];
#pragma unroll
        for (int k = 0; k < kDxTile; k++) {
            const uint32_t li = (uint32_t)raw_i[k];
            const uint32_t alt = li ^ (1u << raw_k[k]);   // minimum-margin bit flipped
            pk[k] = (li * (uint32_t)u.cs.stride) | ((alt * (uint32_t)u.cs.stride) << 16);
            ck[k] = raw_k[k];
        }
        {
            int64_t pb;
            int pdet, pn;
            if (t0 + kDxTile < u.d1) { pb = own_b; pdet = u.cs.det0 + t0 + kDxTile; pn = min(kDxTile, u.d1 - t0 - kDxTile); }
            else if (has_next) { pb = nx.b0 + warp * 32 + lane; pdet = nx.cs.det0 + nx.d0; pn = min(kDxTile, nx.d1 - nx.d0); }
            else { pb = 0; pdet = 0; pn = 0; }
            load_tile_i32<kDxTile>(idx, pb, a.batch, a.n_detectors, pdet, pn, raw_i);
            load_tile_i32<kDxTile>(min_k, pb, a.batch, a.n_detectors, pdet, pn, raw_k);
        }
#pragma unroll
        for (int dd = 0; dd < kDxTile; dd++) {
            if (t0 + dd < u.d1) {
                if (!mbar_wait(ring.full0 + 8 * rp.slot, rp.phase) || *ring.abort_flag) return false;
                if (warp_active) {
                    const float *tab = ring.base + (size_t)rp.slot * a.slot_floats + q;
                    // the lane's own min_delta travels while the products are formed
                    const float own_m = own_b < a.batch ? __ldg(min_delta + own_b * a.n_detectors + u.cs.det0 + t0 + dd) : 0.f;
                    // products of the sample slots i and i + LG/2 are formed together and folded at once (first stage
                    // of the transpose-reduce), so that only LG/2 partial sums stay live
                    float v[LG / 2];
                    const bool top = (j & (LG / 2)) != 0;
#pragma unroll
                    for (int i = 0; i < LG / 2; i++) {
                        const uint32_t pa = __shfl_sync(0xffffffffu, pk[dd], h * LG + i);
                        const uint32_t pb = __shfl_sync(0xffffffffu, pk[dd], h * LG + i + LG / 2);
                        const float va = valid ? gp[i] * (tab[pa & 0xffffu] - tab[pa >> 16]) : 0.f;
                        const float vb = valid ? gp[i + LG / 2] * (tab[pb & 0xffffu] - tab[pb >> 16]) : 0.f;
                        v[i] = (top ? vb : va) + __shfl_xor_sync(0xffffffffu, top ? va : vb, LG / 2);
                    }
                    // remaining stages: after the stage with offset o a lane keeps the half of the values whose index
                    // bit matches its own lane bit, summed with the partner lane's copy
#pragma unroll
                    for (int o = LG / 4; o >= 1; o >>= 1) {
                        const bool upper = (j & o) != 0;
#pragma unroll
                        for (int i = 0; i < o; i++) {
                            const float send = upper ? v[i] : v[i + o];
                            const float keep = upper ? v[i + o] : v[i];
                            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                        }
                    }
                    if (own_b < a.batch) {
                        const double du = surrogate_up(own_m) * (double)v[0];
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
    if (warp == kConsumerWarps) {
        producer_loop(a, ring, lane);
        return;
    }
    int64_t lo, hi;
    block_range(a, &lo, &hi);
    Unit cur, nxt;
    bool has_cur = next_unit(a, lo, hi, cur);
    RingPos rp{0u, 0u};
    int32_t raw_i[kDxTile], raw_k[kDxTile];
    if (has_cur) {
        const int64_t b = cur.b0 + warp * 32 + lane;
        const int det = cur.cs.det0 + cur.d0, n = min(kDxTile, cur.d1 - cur.d0);
        load_tile_i32<kDxTile>(idx, b, a.batch, a.n_detectors, det, n, raw_i);
        load_tile_i32<kDxTile>(min_k, b, a.batch, a.n_detectors, det, n, raw_k);
    }
    while (has_cur) {
        const bool has_next = next_unit(a, cur.next_pos, hi, nxt);
        bool ok;
#define LUTB_DX_UNIT(LGV) \
    input_grad_unit<LGV>(a, cur, nxt, has_next, ring, rp, idx, min_k, min_delta, dY, anchors, raw_i, raw_k, warp, lane, dX)
        if (cur.cs.P <= 8) ok = LUTB_DX_UNIT(8);
        else if (cur.cs.P <= 16) ok = LUTB_DX_UNIT(16);
        else ok = LUTB_DX_UNIT(32);
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
    const size_t tail = 16 * kMaxStages + 128;
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

bool sparse_staged_preferred(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch) {
    // whole tables are streamed whatever the batch: worth it once the batch selects most rows of a table anyway,
    // and when the layer has enough detectors to give every SM a range
    const int64_t rows = (int64_t)1 << cfg->n_anchors;
    return 2 * batch >= rows && cfg->n_detectors >= 4 * device_info().sm_count;
}

static int fill_args(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch, const float *weights,
                     StagedArgs *a, unsigned *grid, size_t *smem) {
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
    int rc = fill_args(cfg, sp, batch, weights, &a, &grid, &smem);
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
    int rc = fill_args(cfg, sp, batch, weights, &a, &grid, &smem);
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
    return LUTB_OK;
}
