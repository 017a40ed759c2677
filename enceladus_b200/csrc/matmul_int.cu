// Exact integer matmul: C[int32] = A @ B with int32 accumulation that wraps modulo 2^32, the semantics of
// an integer tl.dot (src/enceladus/language/ops.py:1255-1259; benchmarks/bench_matmul.py:100-131).
//
// int8 / uint8 operands run on the tcgen05 tensor cores (kind::i8, 128 x BN x 32 per instruction, int32
// accumulators in tensor memory) with the same persistent, warp-specialised pipeline as the floating-point
// kernel: warp 0 feeds a ring of 128-byte-swizzled shared-memory stages by TMA (A 128 rows x 128 K-bytes,
// B 128 K-rows x BN bytes as BN/128 boxes), warp 1 issues the MMAs, warps 2..5 move finished accumulators
// from tensor memory to C while the next tile is being computed.  A is K-major and B is MN-major, so no
// operand is transposed in memory; tiles that hang over an edge rely on TMA zero fill and masked stores.
// 16- and 32-bit integer operands, and 8-bit operands TMA cannot describe, run on a CUDA-core kernel in
// unsigned 32-bit arithmetic (which wraps by definition).
#include "sm100.cuh"

namespace enc {
namespace {

using namespace sm100;

constexpr int BM = 128, BK = 128;  // BK in elements = bytes
constexpr int kThreads = 192;

struct IntMatmulArgs {
    int32_t *c;
    int64_t M, N, K, ldc;
    int is_signed;
    int b_3d;  // the B tensor map is [N/128][K][128]: one copy per stage instead of BN/128
    unsigned *error;
};

template <int BN, int STAGES> struct SmemLayout {
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = BK * BN;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int RING = STAGES * STAGE_BYTES;
    static constexpr int BARRIERS = RING;  // full[S], empty[S], tmem_full[2], tmem_empty[2]
    static constexpr int TOTAL = RING + (2 * STAGES + 4) * 8 + 16;
};

// Instruction descriptor for kind::i8: int32 accumulate (c format 2), A and B both int8 (format 1) or uint8
// (format 0), A K-major, B MN-major, tile M x N.
__host__ __device__ constexpr uint32_t idesc_i8(int is_signed, int m, int n) {
    return (2u << 4) | ((uint32_t)(is_signed ? 1 : 0) << 7) | ((uint32_t)(is_signed ? 1 : 0) << 10) | (1u << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tc_mma_i8_halves(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}

// groups of 16 M-blocks sweep all N-blocks, so the CTAs of one wave share a band of A and a few columns of B in L2
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

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
matmul_i8_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, IntMatmulArgs a) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
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
    constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators of BN int32 columns

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tmem_full[i], 1);
            mbar_init(&tmem_empty[i], 4);  // one arrival per epilogue warp
        }
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
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
                    if (a.b_3d) {
                        tma_load_3d(sb, &tm_b, &full[stage], 0, k * BK, nb * (BN / 128));
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 128; ++j)
                            tma_load_2d(sb + j * (BK * 128), &tm_b, &full[stage], nb * BN + j * 128, k * BK);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (*abort) {  // nobody waits for the copies in flight after an abort: wait here, bounded
                for (uint32_t s = 0; s < (uint32_t)STAGES; ++s) {
                    const uint32_t p = s < stage ? phase : phase ^ 1;
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&full[s], p); ++i) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = idesc_i8(a.is_signed, BM, BN);
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem + L::A_BYTES), BK * 128);  // 128-wide N boxes BK*128 bytes apart
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
                    const uint32_t a_lo = a_lo0 + stage * (L::STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (L::STAGE_BYTES >> 4);
#pragma unroll
                    for (int kk = 0; kk < BK / 32; ++kk)  // 32 K-values: 32 bytes along A's rows, 32 rows (4096 bytes) of B
                        tc_mma_i8_halves(d_tmem, a_lo + kk * (32 >> 4), desc_hi, b_lo + kk * (4096 >> 4), desc_hi, idesc, (k | kk) != 0);
                    tc_commit(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit(&tmem_full[acc]);
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5; TMEM lane quarter = warp % 4) ----------------
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        const bool vec_ok = (a.ldc % 4 == 0) && aligned16(a.c);
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
                if (row < a.M && col < a.N) {
                    int32_t *dst = a.c + row * a.ldc + col;
                    if (vec_ok && col + 32 <= a.N) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<uint4 *>(dst + 4 * i) = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (col + i < a.N) dst[i] = (int32_t)r[i];
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
    if (threadIdx.x == 0 && *abort) atomicExch(a.error, 5u);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- CUDA-core kernel: any integer operand type, any alignment ----------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) matmul_int_simple_kernel(const T *A, const T *B, int32_t *C, int64_t M, int64_t N,
                                                                int64_t K, int64_t lda, int64_t ldb, int64_t ldc) {
    __shared__ uint32_t sa[16][64 + 1], sb[16][64 + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t m0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
    uint32_t acc[4][4] = {};
    for (int64_t k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i / 16, kk = i % 16;
            sa[kk][r] = (m0 + r < M && k0 + kk < K) ? (uint32_t)(int32_t)A[(m0 + r) * lda + k0 + kk] : 0u;  // sign- or zero-extended
            const int kk2 = i / 64, cc = i % 64;
            sb[kk2][cc] = (k0 + kk2 < K && n0 + cc < N) ? (uint32_t)(int32_t)B[(k0 + kk2) * ldb + n0 + cc] : 0u;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            uint32_t av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = sa[kk][ty * 4 + i]; bv[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];  // unsigned: wraps modulo 2^32
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t r = m0 + ty * 4 + i, c = n0 + tx * 4 + j;
            if (r < M && c < N) C[r * ldc + c] = (int32_t)acc[i][j];
        }
}

constexpr int INT_MATMUL_VARIANTS = 2;  // 0: 128x256 tiles, 4 stages; 1: 128x128 tiles, 6 stages

template <int BN, int STAGES>
int launch_tc(const void *A, const void *B, IntMatmulArgs args, int64_t lda, int64_t ldb, cudaStream_t st) {
    using L = SmemLayout<BN, STAGES>;
    char err[256];
    CUtensorMap tm_a, tm_b;
    const uint64_t da[2] = {(uint64_t)args.K, (uint64_t)args.M}, sa[1] = {(uint64_t)lda};
    const uint32_t ba[2] = {BK, BM};
    args.b_3d = args.N % 128 == 0;
    bool ok = make_tensor_map(&tm_a, A, TMAP_U8, 2, da, sa, ba, err, sizeof(err));
    if (ok && args.b_3d) {
        const uint64_t db[3] = {128, (uint64_t)args.K, (uint64_t)(args.N / 128)}, sb[2] = {(uint64_t)ldb, 128};
        const uint32_t bb[3] = {128, BK, BN / 128};
        ok = make_tensor_map(&tm_b, B, TMAP_U8, 3, db, sb, bb, err, sizeof(err));
    } else if (ok) {
        const uint64_t db[2] = {(uint64_t)args.N, (uint64_t)args.K}, sb[1] = {(uint64_t)ldb};
        const uint32_t bb[2] = {128, BK};
        ok = make_tensor_map(&tm_b, B, TMAP_U8, 2, db, sb, bb, err, sizeof(err));
    }
    if (!ok) return fail(ENC_ERR_LAUNCH, "enc_matmul_int: %s", err);
    auto kern = matmul_i8_tc_kernel<BN, STAGES>;
    const int smem = L::TOTAL + 1024;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_matmul_int: cannot opt in to %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    const int64_t tiles = cdiv(args.M, BM) * cdiv(args.N, BN);
    int64_t grid = device_props().sm_count;
    if (grid > tiles) grid = tiles;
    kern<<<(unsigned)grid, kThreads, smem, st>>>(tm_a, tm_b, args);
    return check_launch("enc_matmul_int");
}

template <typename T>
int launch_simple(const void *A, const void *B, const IntMatmulArgs &args, int64_t lda, int64_t ldb, cudaStream_t st) {
    dim3 grid((unsigned)cdiv(args.N, 64), (unsigned)cdiv(args.M, 64));
    if (grid.y > 65535) return fail(ENC_ERR_UNSUPPORTED, "enc_matmul_int: more than 4M rows on the CUDA-core path");
    matmul_int_simple_kernel<T><<<grid, 256, 0, st>>>((const T *)A, (const T *)B, args.c, args.M, args.N, args.K, lda, ldb, args.ldc);
    return check_launch("enc_matmul_int");
}

}  // namespace

int int_matmul_variants() { return INT_MATMUL_VARIANTS; }
void int_matmul_variant_info(int v, char *out, size_t n) {
    snprintf(out, n, "BM=128 BN=%d BK=128 stages=%d tcgen05 kind::i8 (int8/uint8; other integer types: CUDA cores)", v == 0 ? 256 : 128,
             v == 0 ? 4 : 6);
}

}  // namespace enc

extern "C" int enc_matmul_int(const void *a, const void *b, void *c, int64_t M, int64_t N, int64_t K, int64_t lda,
                              int64_t ldb, int64_t ldc, int dtype, int variant, void *stream) {
    ENC_PROLOGUE();
    if (M < 0 || N < 0 || K < 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul_int: negative dimension");
    if (M == 0 || N == 0) return ENC_OK;
    if (!a || !b || !c) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul_int: NULL matrix");
    if (lda < K || ldb < N || ldc < N) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul_int: leading dimension smaller than the row");
    if (variant >= enc::INT_MATMUL_VARIANTS) return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul_int: variant %d out of range", variant);
    cudaStream_t st = enc::as_stream(stream);
    enc::IntMatmulArgs args{static_cast<int32_t *>(c), M, N, K, ldc, dtype == ENC_I8 ? 1 : 0, 0, nullptr};
    if (K == 0) {  // an empty sum: C = 0
        if (cudaMemset2DAsync(c, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, st) != cudaSuccess)
            return enc::fail(ENC_ERR_LAUNCH, "enc_matmul_int: %s", cudaGetErrorString(cudaGetLastError()));
        return ENC_OK;
    }
    switch (dtype) {
        case ENC_I8:
        case ENC_U8: {
            const bool tma_ok = enc::aligned16(a) && enc::aligned16(b) && lda % 16 == 0 && ldb % 16 == 0 && M < (1LL << 31) &&
                                N < (1LL << 31) && K < (1LL << 31);
            if (tma_ok) {
                args.error = enc::device_error_word();
                if (!args.error) return enc::fail(ENC_ERR_NO_MEMORY, "enc_matmul_int: cannot allocate the device status word");
                if (variant < 0) variant = N > 128 ? 0 : 1;
                return variant == 0 ? enc::launch_tc<256, 4>(a, b, args, lda, ldb, st) : enc::launch_tc<128, 6>(a, b, args, lda, ldb, st);
            }
            return dtype == ENC_I8 ? enc::launch_simple<int8_t>(a, b, args, lda, ldb, st)
                                   : enc::launch_simple<uint8_t>(a, b, args, lda, ldb, st);
        }
        case ENC_I16: return enc::launch_simple<int16_t>(a, b, args, lda, ldb, st);
        case ENC_I32: return enc::launch_simple<int32_t>(a, b, args, lda, ldb, st);
        default: return enc::fail(ENC_ERR_BAD_ARG, "enc_matmul_int: dtype %d is not int8, uint8, int16 or int32", dtype);
    }
}
