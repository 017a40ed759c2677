// Inclusive scan (cumsum) for sm_100a.
//
// Flat form (rows == 1): a single pass over the data with decoupled look-back.  The array is cut
// into tiles of THREADS*16 elements; persistent CTAs draw tile numbers from an atomic ticket (so a
// tile only ever waits on tiles that are already running), scan their tile in registers, publish
// the tile aggregate, look back over the predecessors' descriptors to obtain the exclusive prefix,
// publish the inclusive prefix and write the result.  Traffic is one read and one write of the
// array; descriptors are 8 bytes per tile ({flag, value} in one 64-bit word, read and written with
// single relaxed gpu-scope accesses, so no fence is needed).  Every wait on a descriptor is bounded;
// when the bound is hit the kernel raises the device error word and finishes without waiting.
//
// Row form: one CTA per row walks the row tile by tile with a running carry.  The reference scans
// one whole row per tile (examples/10_cumsum.py:17-25); rows here may be any length.
//
// Accumulation follows tl.cumsum (src/enceladus/language/ops.py:2047-2060): integers up to 32 bits in
// 32-bit two's-complement arithmetic (unsigned adds, so the wrap is defined), float16/bfloat16/
// float32 in float32, int64 in int64.
#include <map>
#include <mutex>
#include <vector>

#include "sm100.cuh"

namespace enc {
namespace {

constexpr int QUADS = 4;                 // quads (4 consecutive elements) per thread per tile
constexpr int ITEMS = QUADS * 4;         // elements per thread per tile
constexpr unsigned FLAG_EMPTY = 0, FLAG_AGGREGATE = 1, FLAG_PREFIX = 2;
constexpr unsigned SPIN_LIMIT = 1u << 20;  // polls of one descriptor before giving up
constexpr int LOOK = 4;                    // descriptors inspected per lane per look-back round

// ---- element access ------------------------------------------------------------------------
template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<int> { using type = unsigned; };
template <> struct AccOf<signed char> { using type = unsigned; };
template <> struct AccOf<unsigned char> { using type = unsigned; };
template <> struct AccOf<short> { using type = unsigned; };
template <> struct AccOf<long long> { using type = unsigned long long; };

template <typename T> struct OutOf { using type = T; };
template <> struct OutOf<signed char> { using type = int; };
template <> struct OutOf<unsigned char> { using type = int; };
template <> struct OutOf<short> { using type = int; };

template <typename Acc, typename T> __device__ __forceinline__ Acc to_acc(T v) { return (Acc)v; }
template <> __device__ __forceinline__ float to_acc<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_acc<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ unsigned to_acc<unsigned, signed char>(signed char v) { return (unsigned)(int)v; }
template <> __device__ __forceinline__ unsigned to_acc<unsigned, short>(short v) { return (unsigned)(int)v; }

template <typename T, typename Acc> __device__ __forceinline__ T from_acc(Acc v) { return (T)v; }
template <> __device__ __forceinline__ int from_acc<int, unsigned>(unsigned v) { return (int)v; }
template <> __device__ __forceinline__ __half from_acc<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }

template <typename T, int BYTES> struct alignas(BYTES) Quad { T v[4]; };

template <typename T, typename Acc>
__device__ __forceinline__ void load_quad(const T *p, Acc *a) {
    Quad<T, 4 * sizeof(T)> q = *reinterpret_cast<const Quad<T, 4 * sizeof(T)> *>(p);
#pragma unroll
    for (int e = 0; e < 4; ++e) a[e] = to_acc<Acc, T>(q.v[e]);
}
template <typename T, typename Acc>
__device__ __forceinline__ void store_quad(T *p, const Acc *a) {
    Quad<T, 4 * sizeof(T)> q;
#pragma unroll
    for (int e = 0; e < 4; ++e) q.v[e] = from_acc<T, Acc>(a[e]);
    if constexpr (sizeof(q) == 16) {
        st_stream(p, *reinterpret_cast<const uint4 *>(&q));  // written once, read by nobody here: keep it out of L1
    } else {
        *reinterpret_cast<Quad<T, 4 * sizeof(T)> *>(p) = q;
    }
}

// ---- scan of one tile held in registers ----------------------------------------------------
// v[j][e] is element (j*THREADS + thread)*4 + e of the tile.  On return v holds the inclusive scan
// of the tile (no external prefix); the function returns the tile total to every thread.
template <typename Acc, int THREADS>
__device__ __forceinline__ Acc tile_scan(Acc (&v)[QUADS][4], Acc *sh /* [QUADS * THREADS/32 + 1] */) {
    constexpr int NW = THREADS / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    Acc incl[QUADS];
#pragma unroll
    for (int j = 0; j < QUADS; ++j) {
        v[j][1] += v[j][0]; v[j][2] += v[j][1]; v[j][3] += v[j][2];
        incl[j] = v[j][3];
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
        for (int j = 0; j < QUADS; ++j) {
            const Acc up = __shfl_up_sync(0xffffffffu, incl[j], o);
            if (lane >= o) incl[j] += up;
        }
    }
    Acc before[QUADS];  // sum of the quads of the lanes before me, per slab
#pragma unroll
    for (int j = 0; j < QUADS; ++j) {
        before[j] = __shfl_up_sync(0xffffffffu, incl[j], 1);
        if (lane == 0) before[j] = 0;
    }
    __syncthreads();  // sh may still be read by the previous tile's consumers
    if (lane == 31) {
#pragma unroll
        for (int j = 0; j < QUADS; ++j) sh[j * NW + warp] = incl[j];
    }
    __syncthreads();
    if (warp == 0) {
        // exclusive scan of the QUADS*NW warp totals (slab-major order), K consecutive per lane
        constexpr int K = QUADS * NW / 32;
        Acc loc[K > 0 ? K : 1];
        Acc run = 0;
#pragma unroll
        for (int k = 0; k < K; ++k) { loc[k] = sh[lane * K + k]; run += loc[k]; }
        Acc inc = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const Acc up = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += up;
        }
        Acc ex = __shfl_up_sync(0xffffffffu, inc, 1);  // exclusive = previous lane's inclusive
        if (lane == 0) ex = 0;
#pragma unroll
        for (int k = 0; k < K; ++k) { sh[lane * K + k] = ex; ex += loc[k]; }
        if (lane == 31) sh[QUADS * NW] = inc;  // tile total
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < QUADS; ++j) {
        const Acc base = sh[j * NW + warp] + before[j];  // warps before mine + lanes before me
#pragma unroll
        for (int e = 0; e < 4; ++e) v[j][e] += base;
    }
    return sh[QUADS * NW];
}

// ---- descriptors ---------------------------------------------------------------------------
__device__ __forceinline__ void desc_store(unsigned long long *p, unsigned flag, unsigned value) {
    const unsigned long long w = ((unsigned long long)flag << 32) | value;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long desc_load(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ unsigned bits_of(unsigned v) { return v; }
__device__ __forceinline__ unsigned bits_of(float v) { return __float_as_uint(v); }
template <typename Acc> __device__ __forceinline__ Acc acc_of_bits(unsigned b);
template <> __device__ __forceinline__ unsigned acc_of_bits<unsigned>(unsigned b) { return b; }
template <> __device__ __forceinline__ float acc_of_bits<float>(unsigned b) { return __uint_as_float(b); }

struct FlatArgs {
    const void *in;
    void *out;
    int64_t n;
    const void *seed;
    unsigned long long *desc;  // one word per tile, zeroed before the launch
    unsigned *ticket;          // zeroed before the launch
    unsigned *error;           // device error word (sticky)
    int vec;                   // base pointers aligned for quad accesses
};

template <typename TIn, typename Acc, typename TOut, int THREADS>
__global__ void __launch_bounds__(THREADS) scan_lookback_kernel(FlatArgs a) {
    constexpr int TILE = THREADS * ITEMS;
    constexpr int NW = THREADS / 32;
    __shared__ Acc sh[QUADS * NW + 1];
    __shared__ unsigned s_tile;
    __shared__ Acc s_prefix;
    const TIn *in = reinterpret_cast<const TIn *>(a.in);
    TOut *out = reinterpret_cast<TOut *>(a.out);
    const int64_t ntiles = (a.n + TILE - 1) / TILE;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    for (;;) {
        if (threadIdx.x == 0) s_tile = atomicAdd(a.ticket, 1u);
        __syncthreads();
        const int64_t tile = s_tile;
        if (tile >= ntiles) break;
        const int64_t t0 = tile * TILE;
        const bool full = a.vec && t0 + TILE <= a.n;

        Acc v[QUADS][4];
#pragma unroll
        for (int j = 0; j < QUADS; ++j) {
            const int64_t i0 = t0 + ((int64_t)j * THREADS + threadIdx.x) * 4;
            if (full) {
                load_quad<TIn, Acc>(in + i0, v[j]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) v[j][e] = i0 + e < a.n ? to_acc<Acc, TIn>(in[i0 + e]) : Acc(0);
            }
        }
        const Acc total = tile_scan<Acc, THREADS>(v, sh);

        if (warp == 0) {
            Acc exclusive = 0;
            if (tile == 0) {
                if (a.seed) exclusive = *reinterpret_cast<const Acc *>(a.seed);
                if (lane == 0) desc_store(a.desc, FLAG_PREFIX, bits_of(Acc(exclusive + total)));
            } else {
                if (lane == 0) desc_store(a.desc + tile, FLAG_AGGREGATE, bits_of(total));
                // Look back over 32*LOOK descriptors per round: lane l inspects the LOOK predecessors at
                // distances l*LOOK+1 .. l*LOOK+LOOK, nearest first.  The wave of known prefixes then
                // advances 32*LOOK tiles per L2 round trip, which keeps it ahead of the memory system.
                int64_t look = tile - 1;
                bool done = false;
                while (!done) {
                    unsigned flag[LOOK], bits[LOOK];
#pragma unroll
                    for (int k = 0; k < LOOK; ++k) {
                        const int64_t idx = look - (int64_t)lane * LOOK - k;
                        flag[k] = FLAG_PREFIX;  // "before tile 0" acts as a zero prefix
                        bits[k] = 0;
                        if (idx >= 0) {
                            const unsigned long long w = desc_load(a.desc + idx);
                            flag[k] = (unsigned)(w >> 32);
                            bits[k] = (unsigned)w;
                        }
                    }
#pragma unroll
                    for (int k = 0; k < LOOK; ++k) {
                        const int64_t idx = look - (int64_t)lane * LOOK - k;
                        unsigned spins = 0;
                        while (flag[k] == FLAG_EMPTY) {  // the predecessor is still scanning its tile
                            if (++spins > SPIN_LIMIT) {  // give up: flag the error, stop waiting
                                atomicExch(a.error, 1u);
                                flag[k] = FLAG_PREFIX;
                                bits[k] = 0;
                                break;
                            }
                            if (spins > 8) __nanosleep(20);
                            const unsigned long long w = desc_load(a.desc + idx);
                            flag[k] = (unsigned)(w >> 32);
                            bits[k] = (unsigned)w;
                        }
                    }
                    // my LOOK descriptors, nearest first, up to and including my first PREFIX
                    Acc mine = 0;
                    bool has = false;
#pragma unroll
                    for (int k = 0; k < LOOK; ++k) {
                        if (!has) mine += acc_of_bits<Acc>(bits[k]);
                        has = has || flag[k] == FLAG_PREFIX;
                    }
                    const unsigned has_prefix = __ballot_sync(0xffffffffu, has);
                    const int stop = has_prefix ? __ffs(has_prefix) - 1 : 31;
                    Acc contrib = lane <= stop ? mine : Acc(0);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
                    exclusive += contrib;
                    done = has_prefix != 0;
                    look -= 32 * LOOK;
                }
                if (lane == 0) desc_store(a.desc + tile, FLAG_PREFIX, bits_of(Acc(exclusive + total)));
            }
            if (lane == 0) s_prefix = exclusive;
        }
        __syncthreads();
        const Acc prefix = s_prefix;
#pragma unroll
        for (int j = 0; j < QUADS; ++j) {
            const int64_t i0 = t0 + ((int64_t)j * THREADS + threadIdx.x) * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e) v[j][e] += prefix;
            if (full) {
                store_quad<TOut, Acc>(out + i0, v[j]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (i0 + e < a.n) out[i0 + e] = from_acc<TOut, Acc>(v[j][e]);
            }
        }
    }
}

// ---- flat scan fed by a bulk-copy ring ---------------------------------------------------------
// The look-back of a tile cannot finish before every earlier tile has been loaded and reduced, so a
// tile that is slow to arrive stalls all the tiles behind it, and a CTA that holds its tile in
// registers while it waits issues no new loads: with one tile per CTA the bytes in flight per SM
// (about 100 KB of register file) are too few to ride out those stalls at HBM speed.  Here each
// persistent CTA keeps a ring of SLOTS tiles in shared memory instead:
//   warp 0       producer: draws tile tickets and issues one cp.async.bulk per tile into the ring
//                (completion counted in bytes on the slot's mbarrier), as far ahead as the ring allows;
//   warp 1       aggregator: the moment a tile lands it sums it and publishes the tile aggregate, so a
//                claimed tile never keeps its successors waiting for longer than its own load;
//   warp 2       resolver: obtains each tile's exclusive prefix by look-back over the predecessors'
//                descriptors and publishes the inclusive prefix, so the L2 round trips of the look-back
//                are off the scanners' path;
//   warps 3..10  scanners: take the oldest resolved tile into registers (freeing its slot), scan it,
//                add the prefix and store the result.
// Tiles wait for their prefix in shared memory at no cost in registers, and the producer keeps the
// memory system busy while they wait.
constexpr int RING_SCANNERS = 256, RING_THREADS = RING_SCANNERS + 96, RING_TILE = RING_SCANNERS * ITEMS;

__device__ __forceinline__ void scanner_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(RING_SCANNERS) : "memory"); }
// Barrier of the scanner threads that also ANDs a predicate over them: every scanner leaves with the same answer.
__device__ __forceinline__ bool scanner_all(bool ok) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\tbar.red.and.pred p, 1, %2, q;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(r) : "r"((uint32_t)ok), "n"(RING_SCANNERS) : "memory");
    return r != 0;
}

// tile_scan for the 256 scanner threads of the ring kernel (named barrier 1 instead of the CTA barrier)
template <typename Acc>
__device__ __forceinline__ Acc ring_tile_scan(Acc (&v)[QUADS][4], Acc *sh, int tid) {
    constexpr int NW = RING_SCANNERS / 32;
    const int lane = tid & 31, warp = tid >> 5;
    Acc incl[QUADS];
#pragma unroll
    for (int j = 0; j < QUADS; ++j) {
        v[j][1] += v[j][0]; v[j][2] += v[j][1]; v[j][3] += v[j][2];
        incl[j] = v[j][3];
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
        for (int j = 0; j < QUADS; ++j) {
            const Acc up = __shfl_up_sync(0xffffffffu, incl[j], o);
            if (lane >= o) incl[j] += up;
        }
    }
    Acc before[QUADS];
#pragma unroll
    for (int j = 0; j < QUADS; ++j) {
        before[j] = __shfl_up_sync(0xffffffffu, incl[j], 1);
        if (lane == 0) before[j] = 0;
    }
    // (sh is free: every scanner has passed the barrier at the top of this tile's loop iteration, which it
    // reaches only after its last read of sh for the previous tile)
    if (lane == 31) {
#pragma unroll
        for (int j = 0; j < QUADS; ++j) sh[j * NW + warp] = incl[j];
    }
    scanner_barrier();
    if (warp == 0) {  // QUADS * NW == 32 warp totals in slab-major order: one per lane
        const Acc mine = sh[lane];
        Acc inc = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const Acc up = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += up;
        }
        Acc ex = __shfl_up_sync(0xffffffffu, inc, 1);
        if (lane == 0) ex = 0;
        sh[lane] = ex;
        if (lane == 31) sh[QUADS * NW] = inc;
    }
    scanner_barrier();
#pragma unroll
    for (int j = 0; j < QUADS; ++j) {
        const Acc base = sh[j * NW + warp] + before[j];
#pragma unroll
        for (int e = 0; e < 4; ++e) v[j][e] += base;
    }
    return sh[QUADS * NW];
}

// Windows of 32 tile descriptors the resolver reads per round trip.  Measured at 2^30 int32: 1 -> 86% of the copy
// bandwidth, 2 -> 80%, 4 -> 77%, 8 -> 71%: the nearest predecessors publish last, so wider reads mostly add loads
// and polls of descriptors that a later round trip would have found ready.  (Two or three resolver warps taking
// the ring visits in turn were measured too: 78% and 72% - concurrent look-backs find fewer finished prefixes
// nearby and walk further.  Requesting the next visit's window ahead of time lost as well, 81%: what is read
// early is further from a finished prefix.  Windows of 16 or 8 descriptors: 75% and 56% - more round trips.)
constexpr int RING_LOOK = 1;

// Bounded wait on a ring barrier.  A thread that gives up must not simply leave while the others of its role
// go on to a barrier or a warp shuffle it will never reach: the threads that share a role agree on the outcome
// (scanner_all / __all_sync right after the wait) and leave together.
__device__ __forceinline__ bool ring_wait(uint64_t *bar, uint32_t parity, unsigned *error) {
    for (uint32_t i = 0; i < (1u << 22); ++i)
        if (sm100::mbar_try_wait(bar, parity)) return true;
    atomicExch(error, 5u);
    return false;
}

template <typename TIn, typename Acc, typename TOut>
__global__ void __launch_bounds__(RING_THREADS) scan_ring_kernel(FlatArgs a, int slots) {
    using namespace sm100;
    constexpr int NW = RING_SCANNERS / 32;
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ uint64_t full[16], empty[16], aggd[16], pref[16];
    __shared__ long long slot_tile[16];
    __shared__ Acc slot_agg[16], slot_prefix[16];
    __shared__ Acc sh[QUADS * NW + 1];
    const TIn *in = reinterpret_cast<const TIn *>(a.in);
    TOut *out = reinterpret_cast<TOut *>(a.out);
    const int64_t ntiles = (a.n + RING_TILE - 1) / RING_TILE;
    constexpr uint32_t TILE_BYTES = RING_TILE * sizeof(TIn);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < slots; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&aggd[s], 1);
            mbar_init(&pref[s], 1);
            mbar_init(&empty[s], RING_SCANNERS + 2);  // every scanner thread + aggregator + resolver
        }
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t parity = 1;  // a fresh slot counts as released
            for (;;) {
                if (!ring_wait(&empty[s], parity, a.error)) { slot_tile[s] = ntiles; mbar_arrive(&full[s]); break; }
                const long long tile = atomicAdd(a.ticket, 1u);
                slot_tile[s] = tile;
                if (tile >= ntiles) {  // sentinel: tells the consumers of this CTA to stop
                    mbar_arrive(&full[s]);
                    break;
                }
                const int64_t t0 = tile * RING_TILE;
                if (t0 + RING_TILE <= a.n) {
                    mbar_expect_tx(&full[s], TILE_BYTES);
                    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(smem_u32(ring + (size_t)s * TILE_BYTES)), "l"(in + t0), "r"(TILE_BYTES), "r"(smem_u32(&full[s])) : "memory");
                } else {
                    mbar_arrive(&full[s]);  // ragged last tile: the consumers read it from global memory
                }
                if (++s == slots) { s = 0; parity ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------- aggregator: tile sum, published the moment the tile has landed ----------------
        int s = 0;
        uint32_t parity = 0;
        for (;;) {
            const bool ok = __all_sync(0xffffffffu, ring_wait(&full[s], parity, a.error));
            const long long tile = ok ? slot_tile[s] : ntiles;
            if (tile >= ntiles) {
                if (lane == 0) { slot_tile[s] = ntiles; mbar_arrive(&aggd[s]); }  // pass the sentinel on
                break;
            }
            const int64_t t0 = tile * RING_TILE;
            Acc sum = 0;
            if (t0 + RING_TILE <= a.n) {
                const TIn *src = reinterpret_cast<const TIn *>(ring + (size_t)s * TILE_BYTES);
#pragma unroll 4
                for (int q = lane; q < RING_TILE / 4; q += 32) {
                    Acc t[4];
                    load_quad<TIn, Acc>(src + q * 4, t);
                    sum += (t[0] + t[1]) + (t[2] + t[3]);
                }
            } else {
                for (int64_t i = t0 + lane; i < a.n; i += 32) sum += to_acc<Acc, TIn>(in[i]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) {
                if (tile == 0) {
                    Acc seed = 0;
                    if (a.seed) seed = *reinterpret_cast<const Acc *>(a.seed);
                    desc_store(a.desc, FLAG_PREFIX, bits_of(Acc(seed + sum)));
                } else {
                    desc_store(a.desc + tile, FLAG_AGGREGATE, bits_of(sum));
                }
                slot_agg[s] = sum;
                mbar_arrive(&aggd[s]);
                mbar_arrive(&empty[s]);
            }
            if (++s == slots) { s = 0; parity ^= 1; }
        }
    } else if (warp == 2) {
        // ---------------- resolver: exclusive prefix of each tile by look-back, off the scanners' path ----------------
        int s = 0;
        uint32_t parity = 0;
        for (;;) {
            const bool ok = __all_sync(0xffffffffu, ring_wait(&aggd[s], parity, a.error));
            const long long tile = ok ? slot_tile[s] : ntiles;
            if (tile >= ntiles) {
                if (lane == 0) { slot_tile[s] = ntiles; mbar_arrive(&pref[s]); }
                break;
            }
            Acc exclusive = 0;
            if (tile == 0) {
                if (a.seed) exclusive = *reinterpret_cast<const Acc *>(a.seed);
            } else {
                int64_t look = tile - 1;
                bool done = false;
                while (!done) {
                    // RING_LOOK windows of 32 descriptors per round trip, nearest first
                    unsigned long long w[RING_LOOK];
#pragma unroll
                    for (int k = 0; k < RING_LOOK; ++k) {
                        const int64_t idx = look - 32 * k - lane;
                        w[k] = idx >= 0 ? desc_load(a.desc + idx) : ((unsigned long long)FLAG_PREFIX << 32);
                    }
#pragma unroll
                    for (int k = 0; k < RING_LOOK; ++k) {
                        if (done) break;
                        const int64_t idx = look - 32 * k - lane;
                        unsigned flag = (unsigned)(w[k] >> 32), bits = (unsigned)w[k];
                        unsigned spins = 0;
                        while (flag == FLAG_EMPTY) {  // that tile has not landed yet
                            if (++spins > SPIN_LIMIT) {
                                atomicExch(a.error, 1u);
                                flag = FLAG_PREFIX;
                                bits = 0;
                                break;
                            }
                            __nanosleep(40);
                            const unsigned long long x = desc_load(a.desc + idx);
                            flag = (unsigned)(x >> 32);
                            bits = (unsigned)x;
                        }
                        const unsigned has_prefix = __ballot_sync(0xffffffffu, flag == FLAG_PREFIX);
                        const int stop = has_prefix ? __ffs(has_prefix) - 1 : 31;
                        Acc contrib = lane <= stop ? acc_of_bits<Acc>(bits) : Acc(0);
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
                        exclusive += contrib;
                        done = has_prefix != 0;
                    }
                    look -= 32 * RING_LOOK;
                }
                if (lane == 0) desc_store(a.desc + tile, FLAG_PREFIX, bits_of(Acc(exclusive + slot_agg[s])));
            }
            if (lane == 0) {
                slot_prefix[s] = exclusive;
                mbar_arrive(&pref[s]);
                mbar_arrive(&empty[s]);
            }
            if (++s == slots) { s = 0; parity ^= 1; }
        }
    } else {
        // ---------------- scanners ----------------
        const int tid = threadIdx.x - 96;
        const bool vec_out = a.vec != 0;
        int s = 0;
        uint32_t parity = 0;
        for (;;) {
            if (!scanner_all(ring_wait(&pref[s], parity, a.error))) break;  // all 256 leave, or none
            const long long tile = slot_tile[s];
            if (tile >= ntiles) break;
            const int64_t t0 = tile * RING_TILE;
            const bool whole = t0 + RING_TILE <= a.n;
            const Acc prefix = slot_prefix[s];
            Acc v[QUADS][4];
            if (whole) {
                const TIn *src = reinterpret_cast<const TIn *>(ring + (size_t)s * TILE_BYTES);
#pragma unroll
                for (int j = 0; j < QUADS; ++j) load_quad<TIn, Acc>(src + (j * RING_SCANNERS + tid) * 4, v[j]);
            } else {
#pragma unroll
                for (int j = 0; j < QUADS; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int64_t i = t0 + ((int64_t)j * RING_SCANNERS + tid) * 4 + e;
                        v[j][e] = i < a.n ? to_acc<Acc, TIn>(in[i]) : Acc(0);
                    }
            }
            mbar_arrive(&empty[s]);  // tile and prefix are in registers: the slot can be refilled
            ring_tile_scan<Acc>(v, sh, tid);
#pragma unroll
            for (int j = 0; j < QUADS; ++j) {
                const int64_t i0 = t0 + ((int64_t)j * RING_SCANNERS + tid) * 4;
#pragma unroll
                for (int e = 0; e < 4; ++e) v[j][e] += prefix;
                if (whole && vec_out) {
                    store_quad<TOut, Acc>(out + i0, v[j]);
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (i0 + e < a.n) out[i0 + e] = from_acc<TOut, Acc>(v[j][e]);
                }
            }
            if (++s == slots) { s = 0; parity ^= 1; }
        }
    }
}

// ---- row form ------------------------------------------------------------------------------
struct RowScanArgs {
    const void *in;
    void *out;
    int64_t rows, cols, stride_in, stride_out;
    int reverse;
    int vec;
};

template <typename TIn, typename Acc, typename TOut, int THREADS>
__global__ void __launch_bounds__(THREADS) scan_rows_kernel(RowScanArgs a) {
    constexpr int TILE = THREADS * ITEMS;
    constexpr int NW = THREADS / 32;
    __shared__ Acc sh[QUADS * NW + 1];
    const int64_t row = blockIdx.x;
    const TIn *in = reinterpret_cast<const TIn *>(a.in) + row * a.stride_in;
    TOut *out = reinterpret_cast<TOut *>(a.out) + row * a.stride_out;
    const bool rev = a.reverse != 0;
    Acc carry = 0;
    for (int64_t t0 = 0; t0 < a.cols; t0 += TILE) {
        const bool full = a.vec && !rev && t0 + TILE <= a.cols;
        Acc v[QUADS][4];
#pragma unroll
        for (int j = 0; j < QUADS; ++j) {
            const int64_t i0 = t0 + ((int64_t)j * THREADS + threadIdx.x) * 4;
            if (full) {
                load_quad<TIn, Acc>(in + i0, v[j]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int64_t i = i0 + e;  // position in scan order; mirrored when reversed
                    v[j][e] = i < a.cols ? to_acc<Acc, TIn>(in[rev ? a.cols - 1 - i : i]) : Acc(0);
                }
            }
        }
        const Acc total = tile_scan<Acc, THREADS>(v, sh);
#pragma unroll
        for (int j = 0; j < QUADS; ++j) {
            const int64_t i0 = t0 + ((int64_t)j * THREADS + threadIdx.x) * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e) v[j][e] += carry;
            if (full) {
                store_quad<TOut, Acc>(out + i0, v[j]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int64_t i = i0 + e;
                    if (i < a.cols) out[rev ? a.cols - 1 - i : i] = from_acc<TOut, Acc>(v[j][e]);
                }
            }
        }
        carry += total;
    }
}

// ---- total (pass 1 of the multi-GPU flat scan) ---------------------------------------------
// A pure read at the speed of the memory system: 16-byte streaming loads, four in flight per thread, four
// accumulators.  (Any summation order is allowed: integers wrap, and the float32 total only positions the
// shard's scan, whose tolerance is relative to the exact prefix.)
template <typename TIn, typename Acc>
__device__ __forceinline__ Acc sum_vec16(const uint4 &u) {
    constexpr int PER = 16 / sizeof(TIn);
    const TIn *e = reinterpret_cast<const TIn *>(&u);
    Acc s = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) s += to_acc<Acc, TIn>(e[i]);
    return s;
}

template <typename TIn, typename Acc>
__global__ void __launch_bounds__(256) sum_partials_kernel(const TIn *in, int64_t n, Acc *partials) {
    constexpr int PER = 16 / sizeof(TIn);
    __shared__ Acc sh[8];
    Acc s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nvec = aligned16(in) ? n / PER : 0;
    const uint4 *v = reinterpret_cast<const uint4 *>(in);
    // A CTA reads slabs of 8 x 256 consecutive vectors (32 KB): eight loads in flight per thread, each a fully
    // coalesced 4 KB row of the slab, slabs dealt round-robin to the CTAs.  The slabs are walked from the END of the
    // array towards its beginning: the scan that follows this pass in the multi-GPU recipe starts at the beginning,
    // which is then what L2 still holds.
    constexpr int U = 8;
    const int64_t slab = (int64_t)U * blockDim.x, nslabs = nvec / slab;
    for (int64_t it = blockIdx.x; it < nslabs; it += gridDim.x) {
        const int64_t sl = nslabs - 1 - it;
        const uint4 *p = v + sl * slab + threadIdx.x;
        uint4 q[U];
#pragma unroll
        for (int u = 0; u < U; ++u) q[u] = ld_stream(p + u * blockDim.x);
#pragma unroll
        for (int u = 0; u < U; u += 4) {
            s0 += sum_vec16<TIn, Acc>(q[u]);
            s1 += sum_vec16<TIn, Acc>(q[u + 1]);
            s2 += sum_vec16<TIn, Acc>(q[u + 2]);
            s3 += sum_vec16<TIn, Acc>(q[u + 3]);
        }
    }
    for (int64_t i = nslabs * slab + tid; i < nvec; i += stride) s0 += sum_vec16<TIn, Acc>(ld_stream(v + i));
    for (int64_t j = nvec * PER + tid; j < n; j += stride) s1 += to_acc<Acc, TIn>(in[j]);
    Acc s = (s0 + s1) + (s2 + s3);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        Acc t = 0;
        for (int i = 0; i < 8; ++i) t += sh[i];
        partials[blockIdx.x] = t;
    }
}
template <typename Acc>
__global__ void __launch_bounds__(1024) sum_final_kernel(const Acc *partials, int count, Acc *total) {
    __shared__ Acc sh[32];
    Acc s = 0;
    for (int i = threadIdx.x; i < count; i += blockDim.x) s += partials[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        Acc t = 0;
        for (int i = 0; i < 32; ++i) t += sh[i];
        *total = t;
    }
}

// Exclusive offset of shard `index` from the gathered per-shard totals: totals[0] + ... + totals[index-1] in the
// scan's own arithmetic (unsigned wrap / float32 or int64 adds in shard order).  One thread; it exists so that
// the multi-GPU scan never leaves the stream between its two passes.
template <typename Acc>
__global__ void scan_offset_kernel(const Acc *totals, int index, Acc *out) {
    Acc s = 0;
    for (int i = 0; i < index; ++i) s += totals[i];
    *out = s;
}

// ---- scratch -------------------------------------------------------------------------------
// One buffer per (device, stream): launches on one stream are ordered, so they can share it, and
// launches on different streams never collide.  A stream that is being captured into a CUDA graph
// cannot allocate, and the graph may later be replayed on any stream, so captured launches use one
// extra per-device buffer that every ordinary call keeps at least as large as its own (run the
// same call once before capturing it).  A graph keeps the address it captured in its memset node and
// kernel arguments, so a capture buffer that was ever handed out under capture is never freed or moved:
// when a later ordinary call needs a larger one, the old block is retired (kept until exit) and new
// captures get the larger block.  All captured scans of a device share their block: replay two such
// graphs on different streams at the same time and their descriptors race.
struct Scratch { void *ptr = nullptr; size_t bytes = 0; bool captured = false; };
std::mutex g_scratch_mu;
std::map<std::pair<int, void *>, Scratch> g_scratch;
std::vector<void *> g_retired;  // capture buffers that instantiated graphs may still point at
void *const kCaptureKey = reinterpret_cast<void *>(~uintptr_t(0));

bool grow(Scratch &s, size_t bytes, cudaStream_t st) {
    if (s.bytes >= bytes) return true;
    if (s.ptr) {
        if (s.captured) {
            g_retired.push_back(s.ptr);
        } else {
            cudaStreamSynchronize(st);  // earlier launches may still use it
            cudaFree(s.ptr);
        }
    }
    s.ptr = nullptr;
    s.bytes = 0;
    s.captured = false;
    const size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
    if (cudaMalloc(&s.ptr, want) != cudaSuccess) {
        cudaGetLastError();
        s.ptr = nullptr;
        return false;
    }
    s.bytes = want;
    return true;
}

void *scratch_get(size_t bytes, void *stream) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(as_stream(stream), &cap) != cudaSuccess) cudaGetLastError();
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (cap != cudaStreamCaptureStatusNone) {
        Scratch &c = g_scratch[{dev, kCaptureKey}];
        if (c.bytes < bytes) return nullptr;
        c.captured = true;
        return c.ptr;
    }
    if (!grow(g_scratch[{dev, kCaptureKey}], bytes, nullptr)) return nullptr;
    Scratch &s = g_scratch[{dev, stream}];
    return grow(s, bytes, as_stream(stream)) ? s.ptr : nullptr;
}

// variant v: 0..2 one tile per CTA in registers, CTA threads = {256, 512, 1024}[v] (tile = threads * 16
// elements); 3 = 4096-element tiles through a shared-memory ring fed by the bulk-copy engine
constexpr int SCAN_VARIANTS = 4;
constexpr int kAutoScanVariant = 3;

template <typename TIn>
int launch_flat_ring(const void *in, void *out, int64_t n, const void *seed, cudaStream_t st, void *stream) {
    using Acc = typename AccOf<TIn>::type;
    using TOut = typename OutOf<TIn>::type;
    const int64_t ntiles = cdiv(n, RING_TILE);
    const size_t bytes = 64 + (size_t)ntiles * 8;
    char *scr = (char *)scratch_get(bytes, stream);
    if (!scr) return fail(ENC_ERR_NO_MEMORY, "enc_cumsum: cannot allocate %zu bytes of tile descriptors (inside a stream capture nothing can be allocated: run the same call once before capturing)", bytes);
    unsigned *err = device_error_word();
    if (!err) return fail(ENC_ERR_NO_MEMORY, "enc_cumsum: cannot allocate the device status word");
    cudaError_t e = cudaMemsetAsync(scr, 0, bytes, st);
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_cumsum: memset of descriptors failed: %s", cudaGetErrorString(e));
    FlatArgs a{in, out, n, seed, (unsigned long long *)(scr + 64), (unsigned *)scr, err,
               reinterpret_cast<uintptr_t>(out) % (4 * sizeof(TOut)) == 0 ? 1 : 0};
    const size_t tile_bytes = (size_t)RING_TILE * sizeof(TIn);
    // About 96 KB of tiles per CTA, two CTAs per SM.  Measured at 2^30 int32: throughput follows the bytes the rings
    // hold per SM (2 x 64 KB: 64% of the copy bandwidth, 2 x 96 KB or 3 x 64 KB: 80%), not the number of scanner warps
    // (one CTA with a 192 KB ring: 59%).
    int slots = (int)((96 * 1024) / tile_bytes);
    if (slots > 16) slots = 16;
    if (slots < 2) slots = 2;
    const size_t smem = tile_bytes * slots;
    auto kern = scan_ring_kernel<TIn, Acc, TOut>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_cumsum: cannot opt in to shared memory: %s", cudaGetErrorString(e));
    int64_t grid = (int64_t)device_props().sm_count * 2;
    if (grid > ntiles) grid = ntiles;
    kern<<<(unsigned)grid, RING_THREADS, smem, st>>>(a, slots);
    return check_launch("enc_cumsum");
}

template <typename TIn, int THREADS>
int launch_flat_t(const void *in, void *out, int64_t n, const void *seed, cudaStream_t st, void *stream) {
    using Acc = typename AccOf<TIn>::type;
    using TOut = typename OutOf<TIn>::type;
    constexpr int TILE = THREADS * ITEMS;
    const int64_t ntiles = cdiv(n, TILE);
    const size_t bytes = 64 + (size_t)ntiles * 8;
    char *scr = (char *)scratch_get(bytes, stream);
    if (!scr) return fail(ENC_ERR_NO_MEMORY, "enc_cumsum: cannot allocate %zu bytes of tile descriptors (inside a stream capture nothing can be allocated: run the same call once before capturing)", bytes);
    unsigned *err = device_error_word();
    if (!err) return fail(ENC_ERR_NO_MEMORY, "enc_cumsum: cannot allocate the device status word");
    cudaError_t e = cudaMemsetAsync(scr, 0, bytes, st);
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_cumsum: memset of descriptors failed: %s", cudaGetErrorString(e));
    FlatArgs a{in, out, n, seed, (unsigned long long *)(scr + 64), (unsigned *)scr, err,
               (reinterpret_cast<uintptr_t>(in) % (4 * sizeof(TIn)) == 0 && reinterpret_cast<uintptr_t>(out) % (4 * sizeof(TOut)) == 0) ? 1 : 0};
    int64_t grid = (int64_t)device_props().sm_count * (2048 / THREADS);
    if (grid > ntiles) grid = ntiles;
    scan_lookback_kernel<TIn, Acc, TOut, THREADS><<<(unsigned)grid, THREADS, 0, st>>>(a);
    return check_launch("enc_cumsum");
}

template <typename TIn, int THREADS>
int launch_rows_t(const void *in, void *out, int64_t rows, int64_t cols, int64_t si, int64_t so, int reverse, cudaStream_t st) {
    using Acc = typename AccOf<TIn>::type;
    using TOut = typename OutOf<TIn>::type;
    const bool vec = reinterpret_cast<uintptr_t>(in) % (4 * sizeof(TIn)) == 0 && reinterpret_cast<uintptr_t>(out) % (4 * sizeof(TOut)) == 0 &&
                     si % 4 == 0 && so % 4 == 0;
    RowScanArgs a{in, out, rows, cols, si, so, reverse, vec ? 1 : 0};
    scan_rows_kernel<TIn, Acc, TOut, THREADS><<<(unsigned)rows, THREADS, 0, st>>>(a);
    return check_launch("enc_cumsum");
}

template <typename TIn, bool LOOKBACK>
int launch_scan(const void *in, void *out, int64_t rows, int64_t cols, int64_t si, int64_t so, int reverse,
                const void *seed, int variant, void *stream) {
    cudaStream_t st = as_stream(stream);
    if (rows == 0 || cols == 0) return ENC_OK;
    if constexpr (LOOKBACK) {
        if (rows == 1 && !reverse) {
            int v = variant < 0 ? kAutoScanVariant : variant;
            // the bulk-copy engine needs a 16-byte aligned source; other inputs take the register kernels
            if (v == 3 && !aligned16(in)) v = 1;
            switch (v) {
                case 0: return launch_flat_t<TIn, 256>(in, out, cols, seed, st, stream);
                case 1: return launch_flat_t<TIn, 512>(in, out, cols, seed, st, stream);
                case 2: return launch_flat_t<TIn, 1024>(in, out, cols, seed, st, stream);
                default: return launch_flat_ring<TIn>(in, out, cols, seed, st, stream);
            }
        }
    }
    if (seed) return fail(ENC_ERR_UNSUPPORTED, "enc_cumsum: a seed is supported only for the forward flat form (rows == 1) of 32-bit accumulators");
    if (rows > 0x7fffffffLL) return fail(ENC_ERR_UNSUPPORTED, "enc_cumsum: more than 2^31-1 rows");
    // Short rows use small CTAs so that a row does not idle most of its threads.
    int threads = variant < 0 || variant > 2 ? (cols <= 4096 ? 256 : cols <= 8192 ? 512 : 1024) : (256 << variant);
    switch (threads) {
        case 256: return launch_rows_t<TIn, 256>(in, out, rows, cols, si, so, reverse, st);
        case 512: return launch_rows_t<TIn, 512>(in, out, rows, cols, si, so, reverse, st);
        default: return launch_rows_t<TIn, 1024>(in, out, rows, cols, si, so, reverse, st);
    }
}

template <typename TIn>
int launch_sum(const void *in, void *total, int64_t n, void *stream) {
    using Acc = typename AccOf<TIn>::type;
    cudaStream_t st = as_stream(stream);
    int64_t grid = (int64_t)device_props().sm_count * 8;
    const int64_t need = cdiv(n > 0 ? n : 1, 256 * 8 * (16 / (int64_t)sizeof(TIn)));
    if (grid > need) grid = need;
    Acc *partials = (Acc *)scratch_get((size_t)grid * sizeof(Acc), stream);
    if (!partials) return fail(ENC_ERR_NO_MEMORY, "enc_sum: cannot allocate scratch");
    sum_partials_kernel<TIn, Acc><<<(unsigned)grid, 256, 0, st>>>((const TIn *)in, n, partials);
    sum_final_kernel<Acc><<<1, 1024, 0, st>>>(partials, (int)grid, (Acc *)total);
    return check_launch("enc_sum");
}

// ---- flat scan without any allocation ------------------------------------------------------------
// Some hosts of this library must not allocate device memory when they call it: a framework that has
// handed every byte of the device to its own pool (so cudaMalloc fails or fragments it), a serving loop
// that cannot afford the device-wide synchronisation an allocation implies, code that runs under a
// "no allocation after start-up" rule.  For them the tile descriptors of the look-back scan live in
// this array, which is part of the library image: every GPU that loads the library holds it (1 MiB)
// until the process exits.  Word 0 holds the tile ticket, word 1 a spare status word, the
// descriptors start at word 8.
constexpr int NOALLOC_THREADS = 512;                                   // tile = 8192 elements
constexpr int64_t NOALLOC_MAX_TILES = 131072;                          // => at most 2^30 elements
constexpr int64_t NOALLOC_MAX_ELEMS = NOALLOC_MAX_TILES * NOALLOC_THREADS * ITEMS;
static __device__ __align__(256) unsigned long long g_noalloc_scratch[8 + NOALLOC_MAX_TILES];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address; the address
// is looked up once per device (with that device current) and cached.
std::mutex g_noalloc_mu;
void *g_noalloc_addr[64];

int noalloc_scratch_address(void **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_cumsum_noalloc: no current CUDA device (%s)", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(ENC_ERR_UNSUPPORTED, "enc_cumsum_noalloc: device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_addr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return fail(ENC_ERR_LAUNCH, "enc_cumsum_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
        }
        g_noalloc_addr[dev] = p;
    }
    *out = g_noalloc_addr[dev];
    return ENC_OK;
}

template <typename TIn>
int launch_flat_noalloc(const void *in, void *out, int64_t n, const void *seed, unsigned *status, cudaStream_t st) {
    using Acc = typename AccOf<TIn>::type;
    using TOut = typename OutOf<TIn>::type;
    constexpr int TILE = NOALLOC_THREADS * ITEMS;
    void *base = nullptr;
    const int rc = noalloc_scratch_address(&base);
    if (rc != ENC_OK) return rc;
    const int64_t ntiles = cdiv(n, TILE);
    // The array keeps what the previous call left in it: the ticket and this call's descriptors must be zero.
    cudaError_t e = cudaMemsetAsync(base, 0, (size_t)(8 + ntiles) * 8, st);
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_cumsum_noalloc: clearing the descriptors failed: %s", cudaGetErrorString(e));
    unsigned long long *words = reinterpret_cast<unsigned long long *>(base);
    unsigned *spare = reinterpret_cast<unsigned *>(words + 1);
    FlatArgs a{in, out, n, seed, words + 8, reinterpret_cast<unsigned *>(words), status ? status : spare,
               (reinterpret_cast<uintptr_t>(in) % (4 * sizeof(TIn)) == 0 && reinterpret_cast<uintptr_t>(out) % (4 * sizeof(TOut)) == 0) ? 1 : 0};
    int64_t grid = (int64_t)device_props().sm_count * (2048 / NOALLOC_THREADS);
    if (grid > ntiles) grid = ntiles;
    scan_lookback_kernel<TIn, Acc, TOut, NOALLOC_THREADS><<<(unsigned)grid, NOALLOC_THREADS, 0, st>>>(a);
    return check_launch("enc_cumsum_noalloc");
}

}  // namespace

int scan_variants() { return SCAN_VARIANTS; }
void scan_variant_info(int v, char *out, size_t n) {
    if (v == 3) snprintf(out, n, "tile=%d elements through a cp.async.bulk ring in shared memory (producer + aggregator + 256 scanner threads)", RING_TILE);
    else snprintf(out, n, "cta_threads=%d tile=%d elements held in registers", 256 << v, (256 << v) * ITEMS);
}

void scratch_release_all() {
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    for (auto &kv : g_scratch)
        if (kv.second.ptr) cudaFree(kv.second.ptr);
    g_scratch.clear();
    for (void *p : g_retired) cudaFree(p);
    g_retired.clear();
}

}  // namespace enc

extern "C" int enc_cumsum_out_dtype(int dtype) {
    switch (dtype) {
        case ENC_I8: case ENC_U8: case ENC_I16: return ENC_I32;
        case ENC_F32: case ENC_F16: case ENC_BF16: case ENC_I32: case ENC_I64: return dtype;
        default: return -1;
    }
}

extern "C" int enc_cumsum(const void *in, void *out, int64_t rows, int64_t cols, int64_t stride_in,
                          int64_t stride_out, int reverse, int dtype, const void *seed, int variant,
                          void *stream) {
    ENC_PROLOGUE();
    if (rows < 0 || cols < 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_cumsum: negative shape");
    if ((!in || !out) && rows * cols > 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_cumsum: NULL input or output");
    if (variant >= enc::SCAN_VARIANTS) return enc::fail(ENC_ERR_BAD_ARG, "enc_cumsum: variant %d out of range", variant);
    if (rows > 1 && (stride_in < cols || stride_out < cols)) return enc::fail(ENC_ERR_BAD_ARG, "enc_cumsum: row stride smaller than the row length");
    switch (dtype) {
        case ENC_F32: return enc::launch_scan<float, true>(in, out, rows, cols, stride_in, stride_out, reverse, seed, variant, stream);
        case ENC_F16: return enc::launch_scan<__half, true>(in, out, rows, cols, stride_in, stride_out, reverse, seed, variant, stream);
        case ENC_BF16: return enc::launch_scan<__nv_bfloat16, true>(in, out, rows, cols, stride_in, stride_out, reverse, seed, variant, stream);
        case ENC_I32: return enc::launch_scan<int, true>(in, out, rows, cols, stride_in, stride_out, reverse, seed, variant, stream);
        case ENC_I8: return enc::launch_scan<signed char, true>(in, out, rows, cols, stride_in, stride_out, reverse, seed, variant, stream);
        case ENC_U8: return enc::launch_scan<unsigned char, true>(in, out, rows, cols, stride_in, stride_out, reverse, seed, variant, stream);
        case ENC_I16: return enc::launch_scan<short, true>(in, out, rows, cols, stride_in, stride_out, reverse, seed, variant, stream);
        case ENC_I64: return enc::launch_scan<long long, false>(in, out, rows, cols, stride_in, stride_out, reverse, seed, variant, stream);
        default: return enc::fail(ENC_ERR_BAD_ARG, "enc_cumsum: unsupported dtype %d", dtype);
    }
}

extern "C" int enc_sum(const void *in, void *total, int64_t n, int dtype, void *stream) {
    ENC_PROLOGUE();
    if (!total || (!in && n > 0) || n < 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_sum: bad argument");
    switch (dtype) {
        case ENC_F32: return enc::launch_sum<float>(in, total, n, stream);
        case ENC_F16: return enc::launch_sum<__half>(in, total, n, stream);
        case ENC_BF16: return enc::launch_sum<__nv_bfloat16>(in, total, n, stream);
        case ENC_I32: return enc::launch_sum<int>(in, total, n, stream);
        case ENC_I8: return enc::launch_sum<signed char>(in, total, n, stream);
        case ENC_U8: return enc::launch_sum<unsigned char>(in, total, n, stream);
        case ENC_I16: return enc::launch_sum<short>(in, total, n, stream);
        case ENC_I64: return enc::launch_sum<long long>(in, total, n, stream);
        default: return enc::fail(ENC_ERR_BAD_ARG, "enc_sum: unsupported dtype %d", dtype);
    }
}

extern "C" int enc_scan_offset(const void *totals, int count, int index, void *offset, int dtype, void *stream) {
    ENC_PROLOGUE();
    if (!totals || !offset || count < 0 || index < 0 || index > count) return enc::fail(ENC_ERR_BAD_ARG, "enc_scan_offset: bad argument (count %d, index %d)", count, index);
    cudaStream_t st = enc::as_stream(stream);
    switch (dtype) {
        case ENC_F32: case ENC_F16: case ENC_BF16:
            enc::scan_offset_kernel<float><<<1, 1, 0, st>>>((const float *)totals, index, (float *)offset);
            break;
        case ENC_I32: case ENC_I8: case ENC_U8: case ENC_I16:
            enc::scan_offset_kernel<unsigned><<<1, 1, 0, st>>>((const unsigned *)totals, index, (unsigned *)offset);
            break;
        case ENC_I64:
            enc::scan_offset_kernel<unsigned long long><<<1, 1, 0, st>>>((const unsigned long long *)totals, index, (unsigned long long *)offset);
            break;
        default: return enc::fail(ENC_ERR_BAD_ARG, "enc_scan_offset: unsupported dtype %d", dtype);
    }
    return enc::check_launch("enc_scan_offset");
}

// Flat inclusive scan for callers that are not allowed to allocate device memory (see above).  Nothing
// here calls cudaMalloc / cudaFree or any allocating routine: the tile descriptors live in a 1 MiB array
// inside the library image, which caps the length at 2^30 elements.  The first call on a device looks up
// the array's device address (cudaGetSymbolAddress); make that first call before any stream capture.
// All calls on a device share the array, so two calls that overlap on the GPU (different streams) race;
// calls on one stream are ordered and safe.  `status` (device pointer owned by the caller, may be NULL)
// is set non-zero if a bounded look-back wait ran out, in which case the output is invalid.
extern "C" int enc_cumsum_noalloc(const void *in, void *out, int64_t n, int dtype, const void *seed,
                                  unsigned *status, void *stream) {
    ENC_PROLOGUE();
    if (n < 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_cumsum_noalloc: negative length");
    if (n == 0) return ENC_OK;
    if (!in || !out) return enc::fail(ENC_ERR_BAD_ARG, "enc_cumsum_noalloc: NULL input or output");
    if (n > enc::NOALLOC_MAX_ELEMS)
        return enc::fail(ENC_ERR_UNSUPPORTED, "enc_cumsum_noalloc: %lld elements exceed the built-in scratch, which holds descriptors for at most %lld; use enc_cumsum",
                         (long long)n, (long long)enc::NOALLOC_MAX_ELEMS);
    cudaStream_t st = enc::as_stream(stream);
    switch (dtype) {
        case ENC_F32: return enc::launch_flat_noalloc<float>(in, out, n, seed, status, st);
        case ENC_F16: return enc::launch_flat_noalloc<__half>(in, out, n, seed, status, st);
        case ENC_BF16: return enc::launch_flat_noalloc<__nv_bfloat16>(in, out, n, seed, status, st);
        case ENC_I32: return enc::launch_flat_noalloc<int>(in, out, n, seed, status, st);
        case ENC_I8: return enc::launch_flat_noalloc<signed char>(in, out, n, seed, status, st);
        case ENC_U8: return enc::launch_flat_noalloc<unsigned char>(in, out, n, seed, status, st);
        case ENC_I16: return enc::launch_flat_noalloc<short>(in, out, n, seed, status, st);
        default: return enc::fail(ENC_ERR_UNSUPPORTED, "enc_cumsum_noalloc: dtype %d (32-bit accumulators only: float32/16, bfloat16, int32/16/8, uint8)", dtype);
    }
}
