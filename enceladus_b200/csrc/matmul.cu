// C = epilogue(A @ B) on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of A (128 x 64, K contiguous) and B (64 x BN,
//               N contiguous, as BN/64 boxes of 64 x 64) into a STAGES-deep ring of 128-byte-swizzled
//               shared memory, completion counted in bytes on the stage's "full" mbarrier.  (Prefetching
//               later K blocks into L2 with cp.async.bulk.prefetch.tensor was measured: 20% slower.)
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (128 x BN x 16 per instruction, fp16 or
//               bf16 operands straight from shared memory through matrix descriptors, float32
//               accumulators in tensor memory); tcgen05.commit releases the stage ("empty" mbarrier) and,
//               after the last K block, hands the accumulator to the epilogue ("tmem_full").
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each thread owns one row), add the bias, apply
//               erf-GELU, round to the output type and store 16-byte vectors.  Two accumulator buffers
//               in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
// A is K-major and B is MN-major (row-major [K, N]), so no operand is transposed in memory.  Tiles that
// hang over the matrix edge rely on TMA zero fill for loads and on masked stores, which is the
// descriptor semantics of the reference (src/enceladus/language/ops.py:495-514).  The K loop accumulates
// in float32 in order, as tl.dot does block by block (src/enceladus/language/ops.py:1222-1240).
//
// Operands whose leading dimensions or base addresses are not 16-byte aligned cannot be described to TMA (the
// reference takes such shapes, e.g. 513^3, in its stride: benchmarks/bench_matmul.py:30).  They run the same
// kernel with four extra warps in place of the TMA thread: the loader warps read A and B with plain 32-bit loads
// (any alignment, zero beyond the matrix edge, which is the descriptor semantics) and write them into the stage in
// the 128-byte-swizzled layout the MMA descriptors expect, then make the writes visible to the tensor core's
// proxy and arrive on the stage's "full" barrier.  Nothing is copied or allocated on the way.
#include "sm100.cuh"

namespace enc {
namespace {

using namespace sm100;

constexpr int BM = 128, BK = 64;
constexpr int kThreads = 192;

struct MatmulArgs {
    const void *bias;
    void *c;
    int64_t M, N, K, ldc;
    int epilogue;
    int is_bf16;
    int b_3d;  // the B tensor map is [N/64][K][64]: one copy per stage instead of BN/64
    unsigned *error;
    const void *a_raw, *b_raw;  // loader-warp form only
    int64_t lda, ldb;
};

template <int BN, int STAGES> struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BK * BN * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int RING = STAGES * STAGE_BYTES;
    static constexpr int BARRIERS = RING;                    // full[S], empty[S], tmem_full[2], tmem_empty[2]
    static constexpr int STAGING = RING + (2 * STAGES + 4) * 8 + 16;  // epilogue staging: 4 warps x 32 rows x 17 words
    static constexpr int TOTAL = STAGING + 4 * 32 * 17 * 4;
};

__device__ __forceinline__ float gelu_erf(float t) {
    return __fmul_rn(__fmul_rn(0.5f, t), __fadd_rn(1.0f, erff(__fmul_rn(t, 0.70710677f))));
}

// Tile order: groups of 16 M-blocks sweep all N-blocks, so the CTAs of one wave share a narrow band of A
// and a few columns of B in L2.
__device__ __forceinline__ void tile_coords(int64_t tile, int m_blocks, int n_blocks, int &mb, int &nb) {
    constexpr int GM = 16;
    const int64_t per_group = (int64_t)GM * n_blocks;
    const int group = (int)(tile / per_group);
    const int first = group * GM;
    const int gm = min(GM, m_blocks - first);
    const int in_group = (int)(tile % per_group);
    mb = first + in_group % gm;
    nb = in_group / gm;
}

constexpr int kLoaderThreads = 128;  // MANUAL only: warps 6..9

// One lane's 32-bit word (elements 2*lane and 2*lane+1) of a 64-element row segment that starts at `seg`, which is
// only 2-byte aligned; elements at or beyond `valid` read as zero.  A warp reads the segment's 128 bytes with one
// coalesced instruction when the segment starts on a 4-byte boundary and with two when it does not (the second hits
// the lines the first has fetched); whether it does is the same for the whole warp.  Only aligned words that
// contain at least one valid element are read, so nothing outside the operand's allocation is touched.
// One lane's part of a 64-element row segment that starts at `seg` (2-byte aligned): the aligned word at lane
// offset, and for a segment that starts in the middle of a word the one after it.  p0 / p1 say whether the lane's
// first / second element exists; only aligned words that contain an existing element are read, so nothing
// outside the operand's allocation is touched.  The loads and the combination into the lane's word are separate
// steps and the loads are predicated rather than branched around: a warp executes in order, so an instruction
// that consumes a load's result, or a branch a load cannot be moved across, stalls it once per load instead of
// once per stage (measured: 10 microseconds per stage against one).
struct SegWord { uint32_t x, y; };
__device__ __forceinline__ SegWord load_segment_raw(uintptr_t seg, bool p0, bool p1, int lane, uint32_t &mis_bits, int bit) {
    const uint32_t *w = reinterpret_cast<const uint32_t *>(seg & ~uintptr_t(3)) + lane;
    const bool mis = (seg & 2) != 0;
    mis_bits |= (uint32_t)mis << bit;
    SegWord r;
    // predicated loads into registers that already hold zero: written as PTX so that no select (a consumer of the
    // loaded value, and with it a stall per load) can appear between the loads
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %3, 0;\n\tsetp.ne.b32 q, %4, 0;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\t"
                 "@p ld.global.nc.b32 %0, [%2];\n\t@q ld.global.nc.b32 %1, [%2+4];\n\t}"
                 : "=&r"(r.x), "=&r"(r.y) : "l"(w), "r"((uint32_t)p0), "r"((uint32_t)(mis && p1)));
    return r;  // x: aligned -> both elements, misaligned -> the first one in its high half; y: misaligned -> the second, low half
}
__device__ __forceinline__ uint32_t combine_segment(const SegWord &r, bool mis, bool p1) {
    return mis ? ((r.x >> 16) | (r.y << 16)) : (p1 ? r.x : (r.x & 0xffffu));
}

template <typename T, int BN, int STAGES, bool MANUAL>
__global__ void __launch_bounds__(MANUAL ? kThreads + kLoaderThreads : kThreads, 1)
matmul_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, MatmulArgs a) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // the ring must start on a 1024-byte boundary for the 128-byte swizzle
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L::BARRIERS);
    uint64_t *empty = full + STAGES;
    uint64_t *tmem_full = empty + STAGES;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    volatile uint32_t *abort = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_blocks = (int)((a.M + BM - 1) / BM), n_blocks = (int)((a.N + BN - 1) / BN);
    const int64_t tiles = (int64_t)m_blocks * n_blocks;
    const int k_iters = (int)((a.K + BK - 1) / BK);
    constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators of BN float32 columns

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], MANUAL ? kLoaderThreads : 1);  // every loader thread arrives, or the TMA thread once
            mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tmem_full[i], 1);
            mbar_init(&tmem_empty[i], 4);  // one arrival per epilogue warp
        }
        *abort = 0;
        fence_barrier_init();
        if (!MANUAL) {
            prefetch_tensormap(&tm_a);
            prefetch_tensormap(&tm_b);
        }
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (MANUAL && warp >= 6) {
        // ---------------- loader warps (operands TMA cannot describe) ----------------
        // (Eight loader warps in two groups that fill alternate stages were measured as well: no faster.  At 513^3 the
        // kernel takes 20 microseconds against 6 for the same product from aligned operands; what is left is the
        // latency of one round trip to L2 per stage, which the loader, unlike the TMA unit, does not pipeline across stages.)
        const int lw = warp - 6;  // loader warp 0..3
        // where this lane's word of a 64-element row lands inside the 128-byte swizzled row (XOR with the row added below)
        const uint32_t lane_chunk = lane >> 2, lane_off = (lane & 3) * 4;
        const int e = 2 * lane;  // this lane's first element inside a 64-element segment
        const int64_t step_a = 4 * a.lda * (int64_t)sizeof(T), step_b = 4 * a.ldb * (int64_t)sizeof(T);
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            int mb, nb;
            tile_coords(tile, m_blocks, n_blocks, mb, nb);
            // per tile: rows of A that exist, and which of this lane's two elements exist in each 64-column box of B
            constexpr int NA = BM / 4, NB = BK / 4, NBOX = BN / 64;
            const int rows_left = (int)(a.M - ((int64_t)mb * BM + lw));  // row 4 i + lw exists when 4 i < rows_left
            bool pb0[NBOX], pb1[NBOX];
#pragma unroll
            for (int j = 0; j < NBOX; ++j) {
                const int64_t left = a.N - ((int64_t)nb * BN + j * 64);
                pb0[j] = e < left;
                pb1[j] = e + 1 < left;
            }
            const uintptr_t a_tile = reinterpret_cast<uintptr_t>(a.a_raw) + (((int64_t)mb * BM + lw) * a.lda) * (int64_t)sizeof(T);
            const uintptr_t b_tile = reinterpret_cast<uintptr_t>(a.b_raw) + ((int64_t)lw * a.ldb + (int64_t)nb * BN) * (int64_t)sizeof(T);
            for (int k = 0; k < k_iters && ok; ++k) {
                ok = mbar_wait(&empty[stage], phase ^ 1, abort);
                if (!ok) break;
                uint8_t *sa = smem + stage * L::STAGE_BYTES;
                uint8_t *sb = sa + L::A_BYTES;
                const int64_t k0 = (int64_t)k * BK;
                const int k_left = (int)(a.K - k0);  // K-rows / K-columns of this stage that exist: min(k_left, 64)
                const bool pa0 = e < k_left, pa1 = e + 1 < k_left;
                // A warp takes a row of 64 elements (128 bytes) at a time, one word per lane; pointers advance by
                // addition (a 64-bit multiply per load made the loader instruction bound: 2 microseconds per stage).
                // Every word of the stage is requested before the first one is stored.
                SegWord wa[NA], wb[NB][NBOX];
                uint32_t mis_a = 0, mis_b = 0;
                uintptr_t pa = a_tile + k0 * (int64_t)sizeof(T);
#pragma unroll
                for (int i = 0; i < NA; ++i) {
                    const bool row_ok = 4 * i < rows_left;
                    wa[i] = load_segment_raw(pa, row_ok && pa0, row_ok && pa1, lane, mis_a, i);
                    pa += step_a;
                }
                uintptr_t pb = b_tile + k0 * a.ldb * (int64_t)sizeof(T);
#pragma unroll
                for (int i = 0; i < NB; ++i) {
                    const bool row_ok = 4 * i + lw < k_left;
#pragma unroll
                    for (int j = 0; j < NBOX; ++j)
                        wb[i][j] = load_segment_raw(pb + j * 128, row_ok && pb0[j], row_ok && pb1[j], lane, mis_b, i * NBOX + j);
                    pb += step_b;
                }
#pragma unroll
                for (int i = 0; i < NA; ++i) {
                    const uint32_t r = 4 * i + lw;
                    *reinterpret_cast<uint32_t *>(sa + r * 128 + ((lane_chunk ^ (r & 7)) << 4) + lane_off) =
                        combine_segment(wa[i], (mis_a >> i) & 1, 4 * i < rows_left && pa1);
                }
#pragma unroll
                for (int i = 0; i < NB; ++i) {
                    const uint32_t kr = 4 * i + lw;
#pragma unroll
                    for (int j = 0; j < NBOX; ++j)
                        *reinterpret_cast<uint32_t *>(sb + j * (BK * 128) + kr * 128 + ((lane_chunk ^ (kr & 7)) << 4) + lane_off) =
                            combine_segment(wb[i][j], (mis_b >> (i * NBOX + j)) & 1, (int)kr < k_left && pb1[j]);
                }
                fence_proxy_async();  // generic-proxy writes above -> visible to the tensor core's reads
                mbar_arrive(&full[stage]);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (!MANUAL && lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                int mb, nb;
                tile_coords(tile, m_blocks, n_blocks, mb, nb);
                for (int k = 0; k < k_iters && ok; ++k) {
                    ok = mbar_wait(&empty[stage], phase ^ 1, abort);
                    if (!ok) break;
                    uint8_t *sa = smem + stage * L::STAGE_BYTES;
                    uint8_t *sb = sa + L::A_BYTES;
                    mbar_expect_tx(&full[stage], L::STAGE_BYTES);
                    tma_load_2d(sa, &tm_a, &full[stage], k * BK, mb * BM);
                    if (a.b_3d) {  // one copy: the BN/64 boxes of 64 columns land BK*128 bytes apart, as below
                        tma_load_3d(sb, &tm_b, &full[stage], 0, k * BK, nb * (BN / 64));
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(sb + j * (BK * 128), &tm_b, &full[stage], nb * BN + j * 64, k * BK);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            // Drain: every copy issued above must have landed before the CTA may exit.  The MMA warp
            // normally waits for them; after an abort nobody does, so wait here (bounded) for the most
            // recent fill of every stage.
            if (*abort) {
                for (uint32_t s = 0; s < (uint32_t)STAGES; ++s) {
                    const uint32_t p = s < stage ? phase : phase ^ 1;
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&full[s], p); ++i) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = idesc_f16(a.is_bf16, /*b_mn_major=*/true, BM, BN);
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem + L::A_BYTES), BK * 128);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort);  // epilogue has drained this buffer
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int k = 0; k < k_iters && ok; ++k) {
                    ok = mbar_wait(&full[stage], phase, abort);
                    if (!ok) break;
                    tc_fence_after();
                    // Descriptor low halves: a base per stage plus a constant per step (A: 16 K-values = 32 bytes
                    // further along the swizzled 128-byte rows; B: 16 K-rows = 2048 bytes further, 64-wide N blocks
                    // BK*128 bytes apart).  The issuing thread does as little as possible per MMA.
                    const uint32_t a_lo = a_lo0 + stage * (L::STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (L::STAGE_BYTES >> 4);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)
                        tc_mma_f16_halves(d_tmem, a_lo + kk * (32 >> 4), desc_hi, b_lo + kk * (2048 >> 4), desc_hi, idesc, (k | kk) != 0);
                    tc_commit(&empty[stage]);  // stage reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit(&tmem_full[acc]);  // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5; TMEM lane quarter = warp % 4) ----------------
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        T *c = reinterpret_cast<T *>(a.c);
        const T *bias = reinterpret_cast<const T *>(a.bias);
        const bool vec_ok = (a.ldc % 8 == 0) && aligned16(a.c);
        // rows of C that cannot take 16-byte stores are transposed through these 32 x 32 staging tiles (17-word pitch: no
        // bank conflicts either way), so that a warp writes 64 contiguous bytes of one row per instruction instead of
        // one element in each of 32 rows (which measured 0.3 microseconds per instruction: partial sectors in 32 lines)
        uint32_t *stage_rows = reinterpret_cast<uint32_t *>(smem + L::STAGING) + quarter * (32 * 17);
        for (int64_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            int mb, nb;
            tile_coords(tile, m_blocks, n_blocks, mb, nb);
            ok = mbar_wait(&tmem_full[acc], acc_phase, abort);
            if (!ok) break;
            tc_fence_after();
            const int64_t row = (int64_t)mb * BM + row_in_tile;
            const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(t_row + c0, r);
                tmem_ld_wait();
                const int64_t col = (int64_t)nb * BN + c0;
                if (col < a.N) {  // (the same for the whole warp)
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                    if (a.epilogue == 1) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float b = (col + i < a.N) ? to_f32(__ldg(bias + col + i)) : 0.0f;
                            v[i] = gelu_erf(__fadd_rn(v[i], b));
                        }
                    }
                    if (vec_ok && col + 32 <= a.N) {
                        if (row < a.M) {
                            T *dst = c + row * a.ldc + col;
#pragma unroll
                            for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4 *>(dst + 8 * i) = Pack<T>::pack(v + 8 * i);
                        }
                    } else {
                        uint32_t *mine = stage_rows + lane * 17;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint4 p = Pack<T>::pack(v + 8 * i);
                            mine[4 * i] = p.x, mine[4 * i + 1] = p.y, mine[4 * i + 2] = p.z, mine[4 * i + 3] = p.w;
                        }
                        __syncwarp();
                        const int64_t row0 = (int64_t)mb * BM + quarter * 32;
                        if (col + lane < a.N) {
#pragma unroll 4
                            for (int rr = 0; rr < 32; ++rr)
                                if (row0 + rr < a.M) c[(row0 + rr) * a.ldc + col + lane] = reinterpret_cast<const T *>(stage_rows + rr * 17)[lane];
                        }
                        __syncwarp();
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort) atomicExch(a.error, 2u);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- CUDA-core fallback for operands TMA cannot describe ------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) matmul_simple_kernel(const T *A, const T *B, const T *bias, T *C, int64_t M,
                                                            int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                                            int epilogue) {
    __shared__ float sa[16][64 + 1], sb[16][64 + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t m0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i / 16, kk = i % 16;
            sa[kk][r] = (m0 + r < M && k0 + kk < K) ? to_f32(A[(m0 + r) * lda + k0 + kk]) : 0.0f;
            const int kk2 = i / 64, cc = i % 64;
            sb[kk2][cc] = (k0 + kk2 < K && n0 + cc < N) ? to_f32(B[(k0 + kk2) * ldb + n0 + cc]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = sa[kk][ty * 4 + i]; bv[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t r = m0 + ty * 4 + i, cc = n0 + tx * 4 + j;
            if (r < M && cc < N) {
                float v = acc[i][j];
                if (epilogue == 1) v = gelu_erf(__fadd_rn(v, to_f32(bias[cc])));
                C[r * ldc + cc] = from_f32<T>(v);
            }
        }
}

// variant v -> (BN, STAGES)
struct TileCfg { int bn, stages; };
constexpr TileCfg kTiles[] = {{256, 4}, {128, 6}, {256, 3}, {64, 8}};
constexpr int MATMUL_VARIANTS = 4;

template <typename T, int BN, int STAGES>
int launch_tc(const void *A, const void *B, const MatmulArgs &args, int64_t lda, int64_t ldb, bool tma_ok, cudaStream_t st) {
    using L = SmemLayout<BN, STAGES>;
    char err[256];
    CUtensorMap tm_a, tm_b;
    memset(&tm_a, 0, sizeof(tm_a));
    memset(&tm_b, 0, sizeof(tm_b));
    MatmulArgs largs = args;
    largs.a_raw = A;
    largs.b_raw = B;
    largs.lda = lda;
    largs.ldb = ldb;
    if (tma_ok) {
        const uint64_t da[2] = {(uint64_t)args.K, (uint64_t)args.M}, sa[1] = {(uint64_t)lda * 2};
        const uint32_t ba[2] = {BK, BM};
        // B [K, N] row-major.  When N is a multiple of 64 it is described as [N/64][K][64], so that one copy brings
        // all BN/64 column boxes of a stage (every TMA instruction costs the producer thread tens of cycles);
        // otherwise as [K][N] with one copy per 64-column box (the ragged last box is zero-filled).
        largs.b_3d = args.N % 64 == 0;
        bool ok = make_tensor_map(&tm_a, A, args.is_bf16, 2, da, sa, ba, err, sizeof(err));
        if (ok && largs.b_3d) {
            const uint64_t db[3] = {64, (uint64_t)args.K, (uint64_t)(args.N / 64)}, sb[2] = {(uint64_t)ldb * 2, 128};
            const uint32_t bb[3] = {64, BK, BN / 64};
            ok = make_tensor_map(&tm_b, B, args.is_bf16, 3, db, sb, bb, err, sizeof(err));
        } else if (ok) {
            const uint64_t db[2] = {(uint64_t)args.N, (uint64_t)args.K}, sb[1] = {(uint64_t)ldb * 2};
            const uint32_t bb[2] = {64, BK};
            ok = make_tensor_map(&tm_b, B, args.is_bf16, 2, db, sb, bb, err, sizeof(err));
        }
        if (!ok) return fail(ENC_ERR_LAUNCH, "enc_matmul: %s", err);
    }
    const int smem = L::TOTAL + 1024;
    const int64_t tiles = cdiv(args.M, BM) * cdiv(args.N, BN);
    int64_t grid = device_props().sm_count;
    if (grid > tiles) grid = tiles;
    cudaError_t e;
    if (tma_ok) {
        auto kern = matmul_tc_kernel<T, BN, STAGES, false>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) kern<<<(unsigned)grid, kThreads, smem, st>>>(tm_a, tm_b, largs);
    } else {
        auto kern = matmul_tc_kernel<T, BN, STAGES, true>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) kern<<<(unsigned)grid, kThreads + kLoaderThreads, smem, st>>>(tm_a, tm_b, largs);
    }
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_matmul: cannot opt in to %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    return check_launch("enc_matmul");
}

template <typename T>
int launch_matmul(const void *A, const void *B, MatmulArgs args, int64_t lda, int64_t ldb, int variant, cudaStream_t st) {
    const bool fits = args.K >= 1 && args.M < (1LL << 31) && args.N < (1LL << 31) && args.K < (1LL << 31);
    if (!fits) {
        dim3 grid((unsigned)cdiv(args.N, 64), (unsigned)cdiv(args.M, 64));
        if (grid.y > 65535) return fail(ENC_ERR_UNSUPPORTED, "enc_matmul: more than 4M rows with a dimension of 2^31 or more");
        matmul_simple_kernel<T><<<grid, 256, 0, st>>>((const T *)A, (const T *)B, (const T *)args.bias, (T *)args.c, args.M,
                                                      args.N, args.K, lda, ldb, args.ldc, args.epilogue);
        return check_launch("enc_matmul");
    }
    // what TMA can describe: 16-byte aligned bases and row pitches; everything else goes through the loader warps
    const bool tma_ok = aligned16(A) && aligned16(B) && lda % 8 == 0 && ldb % 8 == 0;
    args.error = device_error_word();
    if (!args.error) return fail(ENC_ERR_NO_MEMORY, "enc_matmul: cannot allocate the device status word");
    if (variant < 0) {
        // the widest tile that still gives most SMs a tile of their own
        const int64_t sms = device_props().sm_count, mb = cdiv(args.M, BM);
        variant = args.N <= 64 ? 3 : (args.N <= 128 ? 1 : 0);
        if (variant == 0 && mb * cdiv(args.N, 256) * 10 < sms * 6) variant = mb * cdiv(args.N, 128) * 10 >= sms * 6 ? 1 : 3;
    }
    if (!tma_ok && (variant == 0 || variant == 2)) variant = 1;  // the loader warps hold a whole stage in registers: tiles up to 128 wide
    switch (variant) {
        case 0: return launch_tc<T, 256, 4>(A, B, args, lda, ldb, tma_ok, st);
        case 1: return launch_tc<T, 128, 6>(A, B, args, lda, ldb, tma_ok, st);
        case 2: return launch_tc<T, 256, 3>(A, B, args, lda, ldb, tma_ok, st);
        default: return launch_tc<T, 64, 8>(A, B, args, lda, ldb, tma_ok, st);
    }
}

}  // namespace

int matmul_variants() { return MATMUL_VARIANTS; }
void matmul_variant_info(int v, char *out, size_t n) {
    snprintf(out, n, "tile=128x%dx64 stages=%d tcgen05 cta_group::1, TMEM accumulators x2", kTiles[v].bn, kTiles[v].stages);
}

}  // namespace enc

extern "C" int enc_matmul(const void *a, const void *b, const void *bias, void *c, int64_t M, int64_t N,
                          int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int epilogue, int dtype, int variant,
                          void *stream) {
    ENC_PROLOGUE();
    if (M < 0 || N < 0 || K < 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul: negative shape");
    if (M == 0 || N == 0) return ENC_OK;
    if (!a || !b || !c) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul: NULL operand");
    if (epilogue != 0 && epilogue != 1) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul: epilogue must be 0 or 1, got %d", epilogue);
    if (epilogue == 1 && !bias) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul: the bias+GELU epilogue needs a bias");
    if (lda < K || ldb < N || ldc < N) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul: a leading dimension is smaller than its row");
    if (variant >= enc::MATMUL_VARIANTS) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul: variant %d out of range", variant);
    if (K == 0) return enc::fail(ENC_ERR_UNSUPPORTED, "enc_matmul: K == 0");
    enc::MatmulArgs args{bias, c, M, N, K, ldc, epilogue, dtype == ENC_BF16 ? 1 : 0, 0, nullptr, nullptr, nullptr, 0, 0};
    cudaStream_t st = enc::as_stream(stream);
    switch (dtype) {
        case ENC_F16: return enc::launch_matmul<__half>(a, b, args, lda, ldb, variant, st);
        case ENC_BF16: return enc::launch_matmul<__nv_bfloat16>(a, b, args, lda, ldb, variant, st);
        case ENC_F32: {
            // float32 operands keep full precision on the CUDA cores (the tensor cores would round them to tf32)
            dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64));
            if (grid.y > 65535) return enc::fail(ENC_ERR_UNSUPPORTED, "enc_matmul: float32 operands with more than 4M rows");
            enc::matmul_simple_kernel<float><<<grid, 256, 0, st>>>((const float *)a, (const float *)b, (const float *)bias,
                                                                   (float *)c, M, N, K, lda, ldb, ldc, epilogue);
            return enc::check_launch("enc_matmul");
        }
        default: return enc::fail(ENC_ERR_UNSUPPORTED, "enc_matmul: dtype %d; matmul takes float16, bfloat16 or float32", dtype);
    }
}
