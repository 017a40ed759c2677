// Flash-attention forward on the tcgen05 tensor cores of sm_100a.
//
// Three kernels share the arithmetic, which follows the reference kernel (examples/08_flash_attention.py:30-70):
// scores scaled after the float32 dot, exp2 of (score - max) with scale * log2 e folded into one multiply,
// P cast to the input dtype before the second dot, a true division by l at the end; masked with -inf outside
// the sequence and above the diagonal.  The running output is rescaled only when the row maximum has grown by
// more than 2^8 since the last rescale (the statistics stay exact: l and the final 1/l use the same reference
// maximum).  lse = ln2 * (m + log2 l) when requested.  Causal launches skip key blocks above the diagonal.
//
//   attention_ts64_kernel  two 128-row query tiles per CTA, 64-key blocks, S / P / O in tensor memory, three
//                          MMA-issuing threads (the default for sequences longer than one tile)
//   attention_ts_kernel    the same with 128-key blocks and one MMA-issuing thread
//   attention_tc_kernel    one 128-row tile per CTA, P through shared memory:
//     S = Q K^T    (128 x 128, A = Q K-major, B = K block K-major)      -> TMEM, double buffered
//     O += P V     (128 x D,   A = P K-major in shared memory, B = V block MN-major) -> TMEM
//     warp 0      TMA producer (Q once, then K0, K1 V0, K2 V1, ... through the ring: the order of consumption)
//     warp 1      MMA issuer; S of block j+1 is issued before P V of block j so that the tensor core
//                 works while the softmax warps are busy with block j
//     warps 2..5  softmax: thread i owns query row i; P is written to shared memory in the swizzled layout
//                 the MMA reads
//
// Shapes these kernels do not take (head_dim other than 64/128, float32 inputs, strides that TMA
// cannot describe) run on a CUDA-core kernel with the same arithmetic.
#include "sm100.cuh"

namespace enc {
namespace {

using namespace sm100;

constexpr int BM = 128, BN = 128;
constexpr int kThreads = 192;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units
constexpr int kStaggerCycles = 1000;  // head start of tile 0 over tile 1 (see the score issuers)
constexpr int kPolyPairs = 8;  // one pair of exponentials in 8 goes to the FMA pipes (measured best among 0, 1/2, 1/4, 1/8, at head_dim 128 and at 64)

struct AttnArgs {
    void *o;
    float *lse;
    int64_t seq, stride_h, stride_m;
    float qk_scale;  // sm_scale * log2(e), rounded to float32 once
    int causal;
    int is_bf16;
    unsigned *error;
};


// 2^x on the FMA pipes, for the share of the exponentials that the special-function unit (16 results per
// clock per SM) has no time for once two softmax warpgroups run side by side: x = i + f with i integer and f
// in [-0.5, 0.5], 2^f by a cubic (max relative error 7.7e-5, below the bfloat16/float16 rounding of P), the
// exponent field adjusted by i.  Inputs below -126 (masked scores) give 2^-126 instead of zero.  See
// exp2_fma_pair below.

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// 2^x for a pair of values on the FMA pipes
__device__ __forceinline__ void exp2_fma_pair(float x0, float x1, float &p0, float &p1) {
    const uint64_t x = f2_pack(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
    const uint64_t t = f2_add(x, f2_pack(12582912.0f, 12582912.0f));
    const uint64_t f = f2_fma(f2_add(t, f2_pack(-12582912.0f, -12582912.0f)), f2_pack(-1.0f, -1.0f), x);
    uint64_t p = f2_fma(f, f2_pack(0.05508868396282196f, 0.05508868396282196f), f2_pack(0.24260404706001282f, 0.24260404706001282f));
    p = f2_fma(p, f, f2_pack(0.6932762265205383f, 0.6932762265205383f));
    p = f2_fma(p, f, f2_pack(0.9999289512634277f, 0.9999289512634277f));
    float t0, t1, q0, q1;
    f2_unpack(t, t0, t1);
    f2_unpack(p, q0, q1);
    p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
    p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

// One row (or one part of a row) of one score block, in registers.  row_mask_max masks and returns the raw
// maximum; row_exp turns the scores into probabilities in place (float32 bit patterns) against the running
// maximum with lazy rescale and adds their sum to `l`.  `alpha` is the factor the accumulator must be scaled by
// (1 when no rescale is due).  POLY_PAIRS = n: one pair of exponentials in n runs on the FMA pipes (0: none).
// `col0` is the global key index of sv[0][0].
template <int NCH>
__device__ __forceinline__ float row_mask_max(uint32_t (&sv)[NCH][32], bool need_mask, int64_t col0, int64_t row, int64_t seq, int causal) {
    if (need_mask) {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int64_t col = col0 + c * 32 + i;
                if (col >= seq || (causal && col > row)) sv[c][i] = __float_as_uint(-INFINITY);
            }
    }
    // two chains of three-input maxima
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            mx0 = max3(mx0, __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
            mx1 = max3(mx1, __uint_as_float(sv[c][i + 2]), __uint_as_float(sv[c][i + 3]));
        }
    return fmaxf(mx0, mx1);
}

template <int NCH, int POLY_PAIRS>
__device__ __forceinline__ void row_exp(uint32_t (&sv)[NCH][32], float qk_scale, float mx_raw, float &m_ref, float &l, float &alpha,
                                        bool &rescale) {
    const float mx = mx_raw * qk_scale;  // the scale is positive, so it commutes with the maximum
    const float m_new = fmaxf(m_ref, mx);
    // rescale only when the maximum moved far enough for exp2(s - m_ref) to risk overflow
    rescale = m_new > m_ref + RESCALE_THRESHOLD;  // also true for the first finite maximum
    alpha = 1.0f;
    if (rescale) {
        alpha = m_ref == -INFINITY ? 0.0f : fast_exp2(m_ref - m_new);
        m_ref = m_new;
    }
    const float neg_m = m_ref == -INFINITY ? 0.0f : -m_ref;
    const uint64_t scale2 = f2_pack(qk_scale, qk_scale), neg_m2 = f2_pack(neg_m, neg_m);
    uint64_t sum0 = f2_pack(0.0f, 0.0f), sum1 = sum0;  // two chains of packed adds
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            float x0, x1, p0, p1;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1])), scale2, neg_m2), x0, x1);
            if (POLY_PAIRS > 0 && ((c * 16 + (i >> 1)) % (POLY_PAIRS > 0 ? POLY_PAIRS : 1)) == POLY_PAIRS / 2) {
                exp2_fma_pair(x0, x1, p0, p1);
            } else {
                p0 = fast_exp2(x0);
                p1 = fast_exp2(x1);
            }
            const uint64_t p2 = f2_pack(p0, p1);
            if (i & 2) sum1 = f2_add(sum1, p2);
            else sum0 = f2_add(sum0, p2);
            sv[c][i] = __float_as_uint(p0);
            sv[c][i + 1] = __float_as_uint(p1);
        }
    float s0, s1;
    f2_unpack(f2_add(sum0, sum1), s0, s1);
    l = l * alpha + (s0 + s1);
}

template <int NCH, int POLY_PAIRS = 0>
__device__ __forceinline__ void softmax_row(uint32_t (&sv)[NCH][32], float qk_scale, bool need_mask, int64_t n0, int64_t row,
                                            int64_t seq, int causal, float &m_ref, float &l, float &alpha, bool &rescale) {
    const float mx_raw = row_mask_max<NCH>(sv, need_mask, n0, row, seq, causal);
    row_exp<NCH, POLY_PAIRS>(sv, qk_scale, mx_raw, m_ref, l, alpha, rescale);
}

// The same with the mask given as a limit: element e of the block (key col0 + e) is masked when e > lim, where
// lim = min(row, seq - 1) - col0 under a causal mask and seq - 1 - col0 otherwise.  One 32-bit compare per element
// against a value that is fixed per row and block; the kernels for sequences below 2^31 use this form.
template <int NCH>
__device__ __forceinline__ float row_mask_max_lim(uint32_t (&sv)[NCH][32], bool need_mask, int lim) {
    if (need_mask) {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (c * 32 + i > lim) sv[c][i] = __float_as_uint(-INFINITY);
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            mx0 = max3(mx0, __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
            mx1 = max3(mx1, __uint_as_float(sv[c][i + 2]), __uint_as_float(sv[c][i + 3]));
        }
    return fmaxf(mx0, mx1);
}

template <int NCH, int POLY_PAIRS = 0>
__device__ __forceinline__ void softmax_row_lim(uint32_t (&sv)[NCH][32], float qk_scale, bool need_mask, int lim, float &m_ref, float &l,
                                                float &alpha, bool &rescale) {
    const float mx_raw = row_mask_max_lim<NCH>(sv, need_mask, lim);
    row_exp<NCH, POLY_PAIRS>(sv, qk_scale, mx_raw, m_ref, l, alpha, rescale);
}

// P row into shared memory in the swizzled K-major layout the MMA reads: 64-wide boxes, 128-byte rows,
// 16-byte chunk index XOR (row & 7).
template <typename T> __device__ __forceinline__ void store_p_row(uint8_t *p_row, int r, const uint32_t (&sv)[4][32]) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint8_t *box = p_row + (c >> 1) * (BM * 128);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            const int chunk = (c & 1) * 4 + q4;
            float pf[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) pf[i] = __uint_as_float(sv[c][q4 * 8 + i]);
            *reinterpret_cast<uint4 *>(box + ((chunk ^ (r & 7)) << 4)) = Pack<T>::pack(pf);
        }
    }
}

template <int D, int STAGES> struct AttnSmem {
    static constexpr int TILE = BM * D * 2;          // one 128-row block of Q, K or V
    static constexpr int Q_OFF = 0;
    static constexpr int KV_OFF = TILE;
    static constexpr int P_OFF = KV_OFF + STAGES * TILE;
    static constexpr int P_BYTES = BM * BN * 2;
    static constexpr int BAR_OFF = P_OFF + P_BYTES;
    static constexpr int NBARS = 1 + 2 * STAGES + 2 + 2 + 1 + 1 + 1;  // q, kv full/empty, s full/empty, p full/empty, o
    static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
};

template <typename T, int D, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, AttnArgs a) {
    using L = AttnSmem<D, STAGES>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *q_full = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *kv_full = q_full + 1;
    uint64_t *kv_empty = kv_full + STAGES;
    uint64_t *s_full = kv_empty + STAGES;  // [2]
    uint64_t *s_empty = s_full + 2;        // [2]
    uint64_t *p_full = s_empty + 2;
    uint64_t *p_empty = p_full + 1;
    uint64_t *o_full = p_empty + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_full + 1);
    volatile uint32_t *abort = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heavy (late) query blocks first when causal, so the tail of the grid is made of short CTAs
    const int qb = a.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
    const int bh = blockIdx.y;
    const int64_t m0 = (int64_t)qb * BM;
    const int64_t kv_hi = a.causal ? (m0 + BM < a.seq ? m0 + BM : a.seq) : a.seq;
    const int nkv = (int)((kv_hi + BN - 1) / BN);
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t S_COL = 0, O_COL = 256;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 128);
        }
        mbar_init(p_full, 128);
        mbar_init(p_empty, 1);
        mbar_init(o_full, 1);
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            mbar_expect_tx(q_full, L::TILE);
#pragma unroll
            for (int b = 0; b < D / 64; ++b) tma_load_3d(smem + L::Q_OFF + b * (BM * 128), &tm_q, q_full, b * 64, (int)m0, bh);
            bool ok = true;
            uint32_t stage = 0, phase = 0;
            // Blocks are fetched in the order the MMA warp consumes them - K0, K1 V0, K2 V1, ... , V(n-1) - so
            // that the slot a V block frees at the end of one step refills with the K block of the step after next
            // while a whole step is still ahead of it.
            for (int it = 0; it < 2 * nkv && ok; ++it) {
                const bool is_v = it == 2 * nkv - 1 || (it != 0 && (it & 1) == 0);
                const int j = it == 0 ? 0 : it == 2 * nkv - 1 ? nkv - 1 : is_v ? (it - 2) >> 1 : (it + 1) >> 1;
                ok = mbar_wait(&kv_empty[stage], phase ^ 1, abort);
                if (!ok) break;
                uint8_t *dst = smem + L::KV_OFF + stage * L::TILE;
                mbar_expect_tx(&kv_full[stage], L::TILE);
                const CUtensorMap *tm = is_v ? &tm_v : &tm_k;
#pragma unroll
                for (int b = 0; b < D / 64; ++b) tma_load_3d(dst + b * (BN * 128), tm, &kv_full[stage], b * 64, j * BN, bh);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (*abort) {  // drain our own copies before the CTA exits
                for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(q_full, 0); ++i) {}
                for (uint32_t s = 0; s < (uint32_t)STAGES; ++s) {
                    const uint32_t p = s < stage ? phase : phase ^ 1;
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&kv_full[s], p); ++i) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc_s = idesc_f16(a.is_bf16, /*b_mn_major=*/false, BM, BN);
            const uint32_t idesc_o = idesc_f16(a.is_bf16, /*b_mn_major=*/true, BM, D);
            const uint32_t sq = smem_u32(smem + L::Q_OFF), sp = smem_u32(smem + L::P_OFF);
            bool ok = mbar_wait(q_full, 0, abort);
            // ring positions in the producer's order: K_j is item 2j-1 (K_0 item 0), V_j item 2j+2 (the last V item 2n-1)
            auto slot = [&](int it, uint32_t &stage, uint32_t &phase) { stage = it % STAGES; phase = (it / STAGES) & 1; };
            auto k_item = [&](int j) { return j == 0 ? 0 : 2 * j - 1; };
            auto v_item = [&](int j) { return 2 * j + 2 < 2 * nkv - 1 ? 2 * j + 2 : 2 * nkv - 1; };
            auto issue_s = [&](int j) -> bool {  // S_j = Q K_j^T into S buffer j & 1
                uint32_t stage, phase;
                slot(k_item(j), stage, phase);
                if (!mbar_wait(&kv_full[stage], phase, abort)) return false;
                if (!mbar_wait(&s_empty[j & 1], ((j >> 1) & 1) ^ 1, abort)) return false;
                tc_fence_after();
                const uint32_t sk = smem_u32(smem + L::KV_OFF + stage * L::TILE);
                const uint32_t d_tmem = tmem_base + S_COL + (j & 1) * BN;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * (BM * 128) + (kk & 3) * 32;  // 64-wide box, then 32 bytes per step
                    tc_mma_f16(d_tmem, smem_desc_sw128(sq + off, 16, 1024), smem_desc_sw128(sk + off, 16, 1024), idesc_s, kk != 0);
                }
                tc_commit(&kv_empty[stage]);
                tc_commit(&s_full[j & 1]);
                return true;
            };
            if (ok && nkv > 0) ok = issue_s(0);
            for (int j = 0; j < nkv && ok; ++j) {
                if (j + 1 < nkv) {
                    ok = issue_s(j + 1);
                    if (!ok) break;
                }
                uint32_t stage, phase;
                slot(v_item(j), stage, phase);
                ok = mbar_wait(&kv_full[stage], phase, abort);
                ok = ok && mbar_wait(p_full, j & 1, abort);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sv = smem_u32(smem + L::KV_OFF + stage * L::TILE);
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint32_t poff = (kk >> 2) * (BM * 128) + (kk & 3) * 32;
                    // V block: 64-wide column boxes BN*128 bytes apart, 16 key rows = 2048 bytes per step
                    tc_mma_f16(tmem_base + O_COL, smem_desc_sw128(sp + poff, 16, 1024),
                               smem_desc_sw128(sv + kk * 2048, BN * 128, 1024), idesc_o, (j | kk) != 0);
                }
                tc_commit(&kv_empty[stage]);
                tc_commit(p_empty);
            }
            if (ok) tc_commit(o_full);
        }
    } else {
        // ---------------- softmax / epilogue warps ----------------
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;  // query row inside the tile == TMEM lane
        const int64_t row = m0 + r;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        uint8_t *p_row = smem + L::P_OFF + r * 128;
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < nkv && ok; ++j) {
            ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_s = tmem_base + lane_addr + S_COL + (j & 1) * BN;
            const int64_t n0 = (int64_t)j * BN;
            const bool need_mask = (n0 + BN > a.seq) || (a.causal && n0 + BN > m0);
            // The whole score row (128 float32) comes into registers with one wait: a TMEM load issued
            // while MMAs are in flight takes on the order of a thousand cycles, so it is paid once per block.
            uint32_t sv[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, sv[c]);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&s_empty[j & 1]);  // S(j) is in registers: the buffer can take S(j+2)
            float alpha;
            bool rescale;
            softmax_row(sv, a.qk_scale, need_mask, n0, row, a.seq, a.causal, m_ref, l, alpha, rescale);
            // P(j-1) V has finished: the P buffer is free and O is quiescent
            ok = mbar_wait(p_empty, (j & 1) ^ 1, abort);
            if (!ok) break;
            tc_fence_after();
            if (j > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + lane_addr + O_COL + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st_32x32(tmem_base + lane_addr + O_COL + c0, v);
                }
                tmem_st_wait();
                tc_fence_before();
            }
            store_p_row<T>(p_row, r, sv);
            fence_proxy_async();  // make the P stores visible to the tensor core
            mbar_arrive(p_full);
        }
        // ---- epilogue: O / l ----
        if (ok && nkv > 0) ok = mbar_wait(o_full, 0, abort);
        if (ok) {
            tc_fence_after();
            T *o = reinterpret_cast<T *>(a.o) + (int64_t)bh * a.stride_h + row * a.stride_m;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                if (nkv > 0) {
                    tmem_ld_32x32(tmem_base + lane_addr + O_COL + c0, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0;
                }
                if (row < a.seq) {
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __fdiv_rn(__uint_as_float(v[i]), l);
#pragma unroll
                    for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4 *>(o + c0 + 8 * i) = Pack<T>::pack(f + 8 * i);
                }
            }
            if (a.lse && row < a.seq) a.lse[(int64_t)bh * a.seq + row] = (m_ref + log2f(l)) * LN2;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort) atomicExch(a.error, 4u);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- two query tiles per CTA, P in tensor memory --------------------------------------------------------
// The softmax of one 128-row tile takes longer than its two matrix products, so with a single tile per
// CTA the tensor core idles most of the time.  This kernel gives every CTA 256 query rows as two
// independent 128-row tiles, each with its own softmax warpgroup, accumulator and score buffer in tensor
// memory: while one warpgroup exponentiates, the tensor core serves the other tile, and every K/V block
// fetched into shared memory is used twice.
//   warpgroup 0   warp 0 = TMA producer, warp 1 = MMA issuer (registers released with setmaxnreg)
//   warpgroup 1   softmax of tile 0          warpgroup 2   softmax of tile 1
// With P staged through shared memory every step moves, per pair of tiles, 256 KB of MMA operands, 64 KB of
// P stores and 64 KB of TMA writes through the shared-memory port: about 3000 cycles at 128 bytes per cycle,
// more than the 2048 cycles of tensor-core work.  Here the softmax threads write P (rounded to the input
// type, two values per 32-bit column) straight back into tensor memory, over the first 64 columns of the
// score block they have just pulled into registers, and P V reads its A operand from there: no P traffic in
// shared memory, no proxy fence, and the room P took goes to a deeper K/V ring.
//   TMEM columns: S0/P0 [0,128)  S1/P1 [128,256)  O0 [256,256+D)  O1 [384,384+D)
//   issue order per K/V block j: P0(j)V, S0(j+1), P1(j)V, S1(j+1).  S_t(j+1) overwrites P_t(j), so it follows
//   P_t(j)V in the (in-order) MMA pipe; its completion also tells the softmax warpgroup that O_t is
//   quiescent, so the softmax side waits on one barrier per step.
constexpr int kThreads2 = 384;

template <int D, int STAGES> struct AttnSmemTs {
    static constexpr int TILE = BM * D * 2;
    static constexpr int Q_OFF = 0;  // 2 query tiles
    static constexpr int KV_OFF = 2 * TILE;
    static constexpr int BAR_OFF = KV_OFF + STAGES * TILE;
    static constexpr int NBARS = 1 + 2 * STAGES + 4 + 1;  // q, kv full/empty, (s_full, p_full) x 2, o
    static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
};

template <typename T> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

template <typename T, int D, int STAGES>
__global__ void __launch_bounds__(kThreads2, 1)
attention_ts_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, AttnArgs a) {
    using L = AttnSmemTs<D, STAGES>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *q_full = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *kv_full = q_full + 1;
    uint64_t *kv_empty = kv_full + STAGES;
    uint64_t *s_full = kv_empty + STAGES;  // [2] one per tile
    uint64_t *p_full = s_full + 2;         // [2]
    uint64_t *o_full = p_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_full + 1);
    volatile uint32_t *abort = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = a.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;  // heavy blocks first
    const int bh = blockIdx.y;
    const int64_t m0 = (int64_t)qb * (2 * BM);
    int nkv_t[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int64_t r0 = m0 + t * BM;
        const int64_t hi = a.causal ? (r0 + BM < a.seq ? r0 + BM : a.seq) : a.seq;
        nkv_t[t] = r0 < a.seq ? (int)((hi + BN - 1) / BN) : 0;
    }
    const int nkv = nkv_t[0] > nkv_t[1] ? nkv_t[0] : nkv_t[1];
    constexpr uint32_t TMEM_COLS = 512;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&p_full[t], 128);
        }
        mbar_init(o_full, 1);
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == 0 && lane == 0) {
            // ---------------- TMA producer: Q tiles, then K0 V0 K1 V1 ... (the order of consumption) ----------------
            mbar_expect_tx(q_full, 2 * L::TILE);
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int b = 0; b < D / 64; ++b)
                    tma_load_3d(smem + L::Q_OFF + t * L::TILE + b * (BM * 128), &tm_q, q_full, b * 64, (int)(m0 + t * BM), bh);
            bool ok = true;
            uint32_t stage = 0, phase = 0;
            for (int it = 0; it < 2 * nkv && ok; ++it) {
                const int j = it >> 1;
                ok = mbar_wait(&kv_empty[stage], phase ^ 1, abort);
                if (!ok) break;
                uint8_t *dst = smem + L::KV_OFF + stage * L::TILE;
                mbar_expect_tx(&kv_full[stage], L::TILE);
                const CUtensorMap *tm = (it & 1) ? &tm_v : &tm_k;
#pragma unroll
                for (int b = 0; b < D / 64; ++b) tma_load_3d(dst + b * (BN * 128), tm, &kv_full[stage], b * 64, j * BN, bh);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (*abort) {  // drain our own copies before the CTA exits
                for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(q_full, 0); ++i) {}
                for (uint32_t s = 0; s < (uint32_t)STAGES; ++s) {
                    const uint32_t p = s < stage ? phase : phase ^ 1;
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&kv_full[s], p); ++i) {}
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc_s = idesc_f16(a.is_bf16, /*b_mn_major=*/false, BM, BN);
            const uint32_t idesc_o = idesc_f16(a.is_bf16, /*b_mn_major=*/true, BM, D);
            bool ok = mbar_wait(q_full, 0, abort);
            auto slot = [&](int it, uint32_t &stage, uint32_t &phase) { stage = it % STAGES; phase = (it / STAGES) & 1; };
            // descriptor halves: the high half is one constant, the low halves are a base plus a constant per step
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t q_lo = smem_desc_lo(smem_u32(smem + L::Q_OFF), 16);
            const uint32_t k_lo = smem_desc_lo(smem_u32(smem + L::KV_OFF), 16);
            const uint32_t v_lo = smem_desc_lo(smem_u32(smem + L::KV_OFF), BN * 128);
            auto mma_s = [&](int t, uint32_t stage) {  // S_t = Q_t K^T
                const uint32_t qa = q_lo + t * (L::TILE >> 4), kb = k_lo + stage * (L::TILE >> 4);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4;  // 64-wide box, then 32 bytes per step
                    tc_mma_f16_halves(tmem_base + t * BN, qa + off, desc_hi, kb + off, desc_hi, idesc_s, kk != 0);
                }
                tc_commit(&s_full[t]);
            };
            auto mma_pv = [&](int t, int j, uint32_t stage) -> bool {  // O_t += P_t V_j, P_t from tensor memory
                if (!mbar_wait(&p_full[t], j & 1, abort)) return false;
                tc_fence_after();
                const uint32_t vb = v_lo + stage * (L::TILE >> 4);
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk)  // 16 keys = 8 packed columns of P, 16 rows = 2048 bytes of V
                    tc_mma_f16_ts_halves(tmem_base + 256 + t * 128, tmem_base + t * BN + kk * 8, vb + kk * (2048 >> 4), desc_hi,
                                         idesc_o, (j | kk) != 0);
                return true;
            };
            uint32_t stage, phase;
            if (ok && nkv > 0) {
                slot(0, stage, phase);
                ok = mbar_wait(&kv_full[stage], phase, abort);
                if (ok) {
                    tc_fence_after();
#pragma unroll
                    for (int t = 0; t < 2; ++t)
                        if (nkv_t[t] > 0) mma_s(t, stage);
                    tc_commit(&kv_empty[stage]);
                }
            }
            for (int j = 0; j < nkv && ok; ++j) {
                uint32_t vstage, kstage = 0;
                slot(2 * j + 1, vstage, phase);
                ok = mbar_wait(&kv_full[vstage], phase, abort);
                if (!ok) break;
                const bool more = j + 1 < nkv;  // then at least one tile takes K(j+1)
                bool k_ready = false;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (!ok) break;
                    if (j < nkv_t[t]) ok = mma_pv(t, j, vstage);
                    if (t == 1 && ok) tc_commit(&kv_empty[vstage]);  // V(j) is free once both products have run
                    if (ok && j + 1 < nkv_t[t]) {
                        if (!k_ready) {
                            slot(2 * j + 2, kstage, phase);
                            ok = mbar_wait(&kv_full[kstage], phase, abort);
                            if (!ok) break;
                            tc_fence_after();
                            k_ready = true;
                        }
                        mma_s(t, kstage);
                    }
                }
                if (!ok) break;
                if (more) tc_commit(&kv_empty[kstage]);
            }
            if (ok) tc_commit(o_full);
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        // ---------------- softmax warpgroups: tile = warpgroup - 1 ----------------
        const int t = (warp >> 2) - 1;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;  // row inside the tile == TMEM lane
        const int64_t row = m0 + t * BM + r;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem_base + lane_addr + t * BN;
        const uint32_t t_o = tmem_base + lane_addr + 256 + t * 128;
        const int my_nkv = nkv_t[t];
        const int64_t tile_m0 = m0 + t * BM;
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < my_nkv && ok; ++j) {
            // S_t(j) complete; the MMA pipe runs in order, so P_t(j-1) V is complete too and O_t is quiescent
            ok = mbar_wait(&s_full[t], j & 1, abort);
            if (!ok) break;
            tc_fence_after();
            const int64_t n0 = (int64_t)j * BN;
            const bool need_mask = (n0 + BN > a.seq) || (a.causal && n0 + BN > tile_m0);
            uint32_t sv[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, sv[c]);
            tmem_ld_wait();
            float alpha;
            bool rescale;
            softmax_row(sv, a.qk_scale, need_mask, n0, row, a.seq, a.causal, m_ref, l, alpha, rescale);
            if (j > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_o + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st_32x32(t_o + c0, v);
                }
            }
            // P_t(j), two values per column, over the first 64 columns of the score block
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int e = 2 * i;  // element inside this half of 64
                    pk[i] = pack_pair<T>(__uint_as_float(sv[2 * h + (e >> 5)][e & 31]), __uint_as_float(sv[2 * h + (e >> 5)][(e & 31) + 1]));
                }
                tmem_st_32x32(t_s + h * 32, pk);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&p_full[t]);
        }
        // ---- epilogue: O_t / l ----
        if (ok && my_nkv > 0) ok = mbar_wait(o_full, 0, abort);
        if (ok && my_nkv > 0) {
            tc_fence_after();
            T *o = reinterpret_cast<T *>(a.o) + (int64_t)bh * a.stride_h + row * a.stride_m;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld_32x32(t_o + c0, v);
                tmem_ld_wait();
                if (row < a.seq) {
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __fdiv_rn(__uint_as_float(v[i]), l);
#pragma unroll
                    for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4 *>(o + c0 + 8 * i) = Pack<T>::pack(f + 8 * i);
                }
            }
            if (a.lse && row < a.seq) a.lse[(int64_t)bh * a.seq + row] = (m_ref + log2f(l)) * LN2;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort) atomicExch(a.error, 4u);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- two query tiles per CTA, 64-key blocks, score products issued ahead ------------------------------------
// With 128-key blocks the score buffer of a tile is also its P buffer, so S_t(j+1) has to follow P_t(j) V in
// the MMA pipe and every softmax warpgroup idles for two matrix products per step.  With 64-key blocks a
// tile's 128 score columns hold two buffers: S_t(j+1) goes into the other one while the softmax of block j
// runs, P_t(j) overwrites the first 32 columns of its own buffer, and the tensor core never waits for a
// softmax that has work queued.  A 128x64x16 MMA runs at two thirds of the rate of a 128x128x16 one, which
// the removed idle time more than pays for.
//   TMEM columns: tile t buffer b at t*128 + b*64 (S, then P in its first 32)   O0 [256,256+D)  O1 [384,384+D)
//   (Two softmax threads per query row - 640 threads, the halves of a row meeting at a named barrier for the row
//   maximum - were measured as well: 1098 against 1173 TFLOP/s, the exchange costs more than the shorter chain saves.)
//   warp 0 = TMA producer, warps 1 and 2 = score issuers of tile 0 and 1 (S_t(j) goes out as soon as K(j) is
//   there and P_t(j-2) V has left the buffer), warp 3 = P V issuer of both tiles; K and V have a ring each
constexpr int BN64 = 64;

template <int D, int STAGES> struct AttnSmem64 {  // STAGES blocks in the K ring and as many in the V ring
    static constexpr int QTILE = BM * D * 2;
    static constexpr int TILE = BN64 * D * 2;  // one 64-key block of K or V
    static constexpr int Q_OFF = 0;            // 2 query tiles
    static constexpr int K_OFF = 2 * QTILE;
    static constexpr int V_OFF = K_OFF + STAGES * TILE;
    static constexpr int BAR_OFF = V_OFF + STAGES * TILE;
    static constexpr int NBARS = 1 + 4 * STAGES + 12 + 1;  // q, k/v full/empty, (s_full, p_full, pv_done) x 2 tiles x 2 buffers, o
    static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
};

template <typename T, int D, int STAGES>
__global__ void __launch_bounds__(kThreads2, 1)
attention_ts64_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, AttnArgs a) {
    using L = AttnSmem64<D, STAGES>;
    constexpr int BNK = BN64;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *q_full = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *k_full = q_full + 1;
    uint64_t *k_empty = k_full + STAGES;
    uint64_t *v_full = k_empty + STAGES;
    uint64_t *v_empty = v_full + STAGES;
    uint64_t *s_full = v_empty + STAGES;  // [tile * 2 + buffer]
    uint64_t *p_full = s_full + 4;
    uint64_t *pv_done = p_full + 4;
    uint64_t *o_full = pv_done + 4;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_full + 1);
    volatile uint32_t *abort = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = a.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;  // heavy blocks first
    const int bh = blockIdx.y;
    const int64_t m0 = (int64_t)qb * (2 * BM);
    int nkv_t[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int64_t r0 = m0 + t * BM;
        const int64_t hi = a.causal ? (r0 + BM < a.seq ? r0 + BM : a.seq) : a.seq;
        nkv_t[t] = r0 < a.seq ? (int)((hi + BNK - 1) / BNK) : 0;
    }
    const int nkv = nkv_t[0] > nkv_t[1] ? nkv_t[0] : nkv_t[1];
    constexpr uint32_t TMEM_COLS = 512;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 2);  // the score issuers of both tiles release a K block
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
            mbar_init(&pv_done[i], 1);
        }
        mbar_init(o_full, 1);
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == 0 && lane == 0) {
            // ---------------- TMA producer ----------------
            mbar_expect_tx(q_full, 2 * L::QTILE);
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int b = 0; b < D / 64; ++b)
                    tma_load_3d(smem + L::Q_OFF + t * L::QTILE + b * (BM * 128), &tm_q, q_full, b * 64, (int)(m0 + t * BM), bh);
            bool ok = true;
            uint32_t ks = 0, kp = 0, vs = 0, vp = 0;  // ring positions
            for (int it = 0; it < 2 * nkv && ok; ++it) {  // K0, K1 V0, K2 V1, ..., V(n-1): the order of consumption
                const bool is_v = it == 2 * nkv - 1 || (it != 0 && (it & 1) == 0);
                const int j = it == 0 ? 0 : it == 2 * nkv - 1 ? nkv - 1 : is_v ? (it - 2) >> 1 : (it + 1) >> 1;
                uint32_t &st = is_v ? vs : ks, &ph = is_v ? vp : kp;
                uint64_t *full = is_v ? &v_full[st] : &k_full[st];
                ok = mbar_wait(is_v ? &v_empty[st] : &k_empty[st], ph ^ 1, abort);
                if (!ok) break;
                uint8_t *dst = smem + (is_v ? L::V_OFF : L::K_OFF) + st * L::TILE;
                mbar_expect_tx(full, L::TILE);
                const CUtensorMap *tm = is_v ? &tm_v : &tm_k;
#pragma unroll
                for (int b = 0; b < D / 64; ++b) tma_load_3d(dst + b * (BNK * 128), tm, full, b * 64, j * BNK, bh);
                if (++st == STAGES) { st = 0; ph ^= 1; }
            }
            if (*abort) {  // drain our own copies before the CTA exits
                for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(q_full, 0); ++i) {}
                for (uint32_t s = 0; s < (uint32_t)STAGES; ++s) {
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&k_full[s], s < ks ? kp : kp ^ 1); ++i) {}
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&v_full[s], s < vs ? vp : vp ^ 1); ++i) {}
                }
            }
        } else if ((warp == 1 || warp == 2) && lane == 0) {
            // ---------------- score issuers: warp 1 serves tile 0, warp 2 tile 1 ----------------
            // An MMA costs its issuing thread 50-100 cycles next to the busy softmax warps, about what the tensor
            // core needs to execute it, so the three matrix-product streams (S of either tile, P V of both) each
            // get a thread on a scheduler of their own.  Both score issuers walk every K block, waiting for it and
            // releasing it, so that the ring sees two arrivals per block whatever each tile needs.
            const int t = warp - 1;
            const int my_nkv = nkv_t[t];
            const uint32_t idesc_s = idesc_f16(a.is_bf16, /*b_mn_major=*/false, BM, BNK);
            bool ok = mbar_wait(q_full, 0, abort);
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t q_lo = smem_desc_lo(smem_u32(smem + L::Q_OFF + t * L::QTILE), 16);
            const uint32_t k_lo = smem_desc_lo(smem_u32(smem + L::K_OFF), 16);
            const uint32_t s_tmem = tmem_base + t * 128;
            uint32_t stage = 0, phase = 0;
            if (t == 1) {
                // Start tile 1 about half a block period after tile 0, so that the two softmax warpgroups take
                // turns on the special-function unit instead of meeting there; the offset then persists because
                // both tiles do the same work per block.
                const long long t_start = clock64();
                while (clock64() - t_start < kStaggerCycles) {}
            }
            for (int j = 0; j < nkv && ok; ++j) {
                ok = mbar_wait(&k_full[stage], phase, abort);
                if (!ok) break;
                if (j < my_nkv) {
                    // buffer j & 1 held S_t(j-2), then P_t(j-2): free once P_t(j-2) V has completed
                    if (j >= 2) ok = mbar_wait(&pv_done[t * 2 + (j & 1)], ((j - 2) >> 1) & 1, abort);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t kb = k_lo + stage * (L::TILE >> 4);
                    const uint32_t d_tmem = s_tmem + (j & 1) * BNK;
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk)  // 64-wide boxes (128 query rows / 64 key rows each), then 32 bytes per step
                        tc_mma_f16_halves(d_tmem, q_lo + (((kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4), desc_hi,
                                          kb + (((kk >> 2) * (BNK * 128) + (kk & 3) * 32) >> 4), desc_hi, idesc_s, kk != 0);
                    tc_commit(&s_full[t * 2 + (j & 1)]);
                }
                tc_commit(&k_empty[stage]);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        } else if (warp == 3 && lane == 0) {
            // ---------------- P V issuer, both tiles in turn ----------------
            const uint32_t idesc_o = idesc_f16(a.is_bf16, /*b_mn_major=*/true, BM, D);
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t v_lo = smem_desc_lo(smem_u32(smem + L::V_OFF), BNK * 128);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int j = 0; j < nkv && ok; ++j) {
                ok = mbar_wait(&v_full[stage], phase, abort);
                if (!ok) break;
                const uint32_t vb = v_lo + stage * (L::TILE >> 4);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (j >= nkv_t[t]) continue;
                    ok = mbar_wait(&p_full[t * 2 + (j & 1)], (j >> 1) & 1, abort);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t p_tmem = tmem_base + t * 128 + (j & 1) * BNK;
#pragma unroll
                    for (int kk = 0; kk < BNK / 16; ++kk)  // 16 keys = 8 packed columns of P, 16 rows = 2048 bytes of V
                        tc_mma_f16_ts_halves(tmem_base + 256 + t * 128, p_tmem + kk * 8, vb + kk * (2048 >> 4), desc_hi, idesc_o, (j | kk) != 0);
                    tc_commit(&pv_done[t * 2 + (j & 1)]);
                }
                if (!ok) break;
                tc_commit(&v_empty[stage]);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) tc_commit(o_full);
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        // ---------------- softmax warpgroups: tile = warpgroup - 1 ----------------
        const int t = (warp >> 2) - 1;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;  // row inside the tile == TMEM lane
        const int64_t row = m0 + t * BM + r;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem_base + lane_addr + t * 128;
        const uint32_t t_o = tmem_base + lane_addr + 256 + t * 128;
        const int my_nkv = nkv_t[t];
        const int64_t tile_m0 = m0 + t * BM;
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        // block bookkeeping in 32 bits (this kernel takes sequences below 2^31): a block needs its mask when it reaches
        // past `bound`; `last` is the last key this row sees
        const int seq_i = (int)a.seq;
        const int bound = a.causal && (int)tile_m0 < seq_i ? (int)tile_m0 : seq_i;
        const int last_i = a.causal && row < a.seq ? (int)row : seq_i - 1;
        for (int j = 0; j < my_nkv && ok; ++j) {
            const int b = j & 1;
            ok = mbar_wait(&s_full[t * 2 + b], (j >> 1) & 1, abort);
            if (!ok) break;
            tc_fence_after();
            const int n0 = j * BNK;
            const bool need_mask = n0 + BNK > bound;
            uint32_t sv[2][32];
#pragma unroll
            for (int c = 0; c < 2; ++c) tmem_ld_32x32(t_s + b * BNK + c * 32, sv[c]);
            tmem_ld_wait();
            float alpha;
            bool rescale;
            softmax_row_lim<2, kPolyPairs>(sv, a.qk_scale, need_mask, last_i - n0, m_ref, l, alpha, rescale);
            if (j > 0 && __any_sync(0xffffffffu, rescale)) {
                // O_t must be quiescent: P_t(j-1) V complete (P_t(j) V is not issued before this thread's arrival below)
                ok = mbar_wait(&pv_done[t * 2 + (b ^ 1)], ((j - 1) >> 1) & 1, abort);
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_o + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st_32x32(t_o + c0, v);
                }
            }
            // P_t(j), two values per column, over the first 32 columns of its own score buffer
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int e = 2 * i;
                pk[i] = pack_pair<T>(__uint_as_float(sv[e >> 5][e & 31]), __uint_as_float(sv[e >> 5][(e & 31) + 1]));
            }
            tmem_st_32x32(t_s + b * BNK, pk);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&p_full[t * 2 + b]);
        }
        // ---- epilogue: O_t / l ----
        if (ok && my_nkv > 0) ok = mbar_wait(o_full, 0, abort);
        if (ok && my_nkv > 0) {
            tc_fence_after();
            T *o = reinterpret_cast<T *>(a.o) + (int64_t)bh * a.stride_h + row * a.stride_m;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld_32x32(t_o + c0, v);
                tmem_ld_wait();
                if (row < a.seq) {
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __fdiv_rn(__uint_as_float(v[i]), l);
#pragma unroll
                    for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4 *>(o + c0 + 8 * i) = Pack<T>::pack(f + 8 * i);
                }
            }
            if (a.lse && row < a.seq) a.lse[(int64_t)bh * a.seq + row] = (m_ref + log2f(l)) * LN2;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort) atomicExch(a.error, 4u);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- persistent form of the 64-key-block kernel ---------------------------------------------------------------
// The kernel above pays, per 256 query rows, for a CTA launch, barrier set-up, a TMEM allocation, the first Q / K
// loads with nothing to overlap them, and an epilogue during which the tensor core has nothing queued: measured
// from the full and the causal timings at [8, 32, 4096, 128], about 8 microseconds per CTA against 66 (full) or
// 40 (causal) in total.  Here one CTA per SM walks a static list of work items (256 query rows of one (batch,
// head) slice each); barriers and tensor memory are set up once, every ring and every barrier phase simply keeps
// counting across items, and the roles run ahead of each other as far as the data allows:
//   producer       loads the next item's Q tiles as soon as the score products of the current item have read them
//                  (q_empty, committed behind the last score MMA) and keeps the K / V rings full across the seam;
//   score issuers  issue S(0), S(1) of the next item while the softmax warps are still in the epilogue;
//   P V issuer     starts the next item's accumulation once both softmax warpgroups have pulled O out of tensor memory
//                  (o_empty, waited for once per item, outside its block loop; o_full is committed once per item
//                  behind the last product).  Its block loop is the one-shot kernel's, with the buffer parity taken
//                  from a per-tile block count carried across items: per-tile completion barriers and tests for an
//                  item's first and last block inside that loop were measured and cost 10% of the kernel, because
//                  every instruction this thread spends between two products delays the tensor core.
// Schedule: item k = (slice k / n_qb, query block perm[k % n_qb]); CTA c takes k = r G + c in even rounds r and
// k = r G + (G-1-c) in odd ones.  Consecutive items share a slice, so the CTAs of a round read a few slices' K / V
// from L2 as the one-shot grid does.  For causal launches `perm` pairs the query blocks so that the two items a
// CTA gets in an even/odd pair of rounds have a constant total number of key blocks (the host builds it from
// (G, n_qb); see balance_perm16): 98.8% balance for 4096 items on 148 SMs, with no work counter in global memory.
// (The schedule travels as plain scalar kernel parameters, which the hardware reads as constant-bank operands.  A
// struct parameter whose address is taken - a reference to it, a pointer to a table inside it - is read through
// generic loads instead, a few hundred cycles each, and the loops below re-read their parameters after every
// barrier wait: that alone cost 18% when first measured.)
struct Sched {
    int n_qb;         // query blocks of 256 rows per slice
    int n_items;      // n_qb * slices
    uint64_t perm16;  // query-block order inside a slice, 4 bits per position (identity when n_qb > 16)
};

// Work item of this CTA in round r: false when the round has none for it.  The round loop of every role has a
// trip count that depends on kernel parameters and the grid only, and a failed wait skips the remaining rounds
// with `continue` instead of leaving the loop: that keeps r, and everything derived from it (slice, query block,
// row offsets, key-block counts), uniform in the compiler's eyes, so that it lives in uniform registers as the
// blockIdx-derived values of the one-shot kernel do.  (With a `while (ok && next())` loop none of it was, and the
// softmax loop lost 12% to the extra vector registers and instructions.)
__device__ __forceinline__ bool item_of_round(int r, int n_items, int n_qb, uint64_t perm16, int &bh, int &qb) {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const int k = r * G + ((r & 1) ? G - 1 - c : c);
    if (k >= n_items) return false;
    bh = k / n_qb;
    const int q = k - bh * n_qb;
    qb = n_qb <= 16 ? (int)((perm16 >> (4 * q)) & 15) : q;
    return true;
}

// key blocks of 64 the two tiles of query block qb need
__device__ __forceinline__ void item_extent(const AttnArgs &a, int qb, int64_t &m0, int (&nkv_t)[2], int &nkv) {
    m0 = (int64_t)qb * (2 * BM);
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int64_t r0 = m0 + t * BM;
        const int64_t hi = a.causal ? (r0 + BM < a.seq ? r0 + BM : a.seq) : a.seq;
        nkv_t[t] = r0 < a.seq ? (int)((hi + BN64 - 1) / BN64) : 0;
    }
    nkv = nkv_t[0] > nkv_t[1] ? nkv_t[0] : nkv_t[1];
}

template <int D, int STAGES> struct AttnSmemP {  // like AttnSmem64, with per-tile Q and O barriers
    static constexpr int QTILE = BM * D * 2;
    static constexpr int TILE = BN64 * D * 2;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = 2 * QTILE;
    static constexpr int V_OFF = K_OFF + STAGES * TILE;
    static constexpr int BAR_OFF = V_OFF + STAGES * TILE;
    static constexpr int NBARS = 4 + 4 * STAGES + 12 + 4;  // q full/empty x2, k/v full/empty, (s_full, p_full, pv_done) x4, o full/empty x2
    static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
};

template <typename T, int D, int STAGES>
__global__ void __launch_bounds__(kThreads2, 1)
attention_p64_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, AttnArgs a, Sched sc) {
    using L = AttnSmemP<D, STAGES>;
    constexpr int BNK = BN64;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *q_full = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);  // [2]
    uint64_t *q_empty = q_full + 2;                                      // [2]
    uint64_t *k_full = q_empty + 2;
    uint64_t *k_empty = k_full + STAGES;
    uint64_t *v_full = k_empty + STAGES;
    uint64_t *v_empty = v_full + STAGES;
    uint64_t *s_full = v_empty + STAGES;  // [tile * 2 + buffer]
    uint64_t *p_full = s_full + 4;
    uint64_t *pv_done = p_full + 4;
    uint64_t *o_full = pv_done + 4;       // both accumulators complete (committed behind an item's last product)
    uint64_t *o_empty = o_full + 1;       // both softmax warpgroups have pulled their accumulator out of tensor memory
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_empty + 1);
    volatile uint32_t *abort = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t TMEM_COLS = 512;
    const int rounds = (sc.n_items + (int)gridDim.x - 1) / (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int t = 0; t < 2; ++t) {
            mbar_init(&q_full[t], 1);
            mbar_init(&q_empty[t], 1);
        }
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 2);  // the score issuers of both tiles release a K block
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
            mbar_init(&pv_done[i], 1);
        }
        mbar_init(o_full, 1);
        mbar_init(o_empty, 256);
        *abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        // Register budget: the CTA's pool is what it was launched with, 384 threads x 168 registers.  setmaxnreg.inc blocks
        // until the pool has the registers, for ever if it never can: 128 x dec + 256 x inc must not exceed 384 x 168,
        // i.e. dec + 2 inc <= 504.  The persistent producer / issuer loops do not fit in 56 registers (they spilled,
        // and a spill reload in front of every MMA showed up as 7% less tensor-pipe activity): 72 + 2 x 216 = 504.
        static_assert(72 + 2 * 216 <= 3 * 168, "setmaxnreg budget");
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        if (warp == 0 && lane == 0) {
            // ---------------- TMA producer ----------------
            bool ok = true;
            uint32_t ks = 0, kp = 0, vs = 0, vp = 0;  // ring positions
            uint32_t n_q = 0;                         // items whose Q tiles have been requested
            for (int r = 0; r < rounds; ++r) {
                int bh, qb;
                if (!item_of_round(r, sc.n_items, sc.n_qb, sc.perm16, bh, qb) || !ok) continue;
                int64_t m0;
                int nkv_t[2], nkv;
                item_extent(a, qb, m0, nkv_t, nkv);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    ok = ok && mbar_wait(&q_empty[t], (n_q & 1) ^ 1, abort);  // the previous item's score products have read Q_t
                    if (!ok) break;
                    mbar_expect_tx(&q_full[t], L::QTILE);
#pragma unroll
                    for (int b = 0; b < D / 64; ++b)
                        tma_load_3d(smem + L::Q_OFF + t * L::QTILE + b * (BM * 128), &tm_q, &q_full[t], b * 64, (int)(m0 + t * BM), bh);
                }
                if (!ok) continue;
                ++n_q;
                for (int it = 0; it < 2 * nkv && ok; ++it) {  // K0, K1 V0, K2 V1, ..., V(n-1): the order of consumption
                    const bool is_v = it == 2 * nkv - 1 || (it != 0 && (it & 1) == 0);
                    const int j = it == 0 ? 0 : it == 2 * nkv - 1 ? nkv - 1 : is_v ? (it - 2) >> 1 : (it + 1) >> 1;
                    uint32_t &st = is_v ? vs : ks, &ph = is_v ? vp : kp;
                    uint64_t *full = is_v ? &v_full[st] : &k_full[st];
                    ok = mbar_wait(is_v ? &v_empty[st] : &k_empty[st], ph ^ 1, abort);
                    if (!ok) break;
                    uint8_t *dst = smem + (is_v ? L::V_OFF : L::K_OFF) + st * L::TILE;
                    mbar_expect_tx(full, L::TILE);
                    const CUtensorMap *tm = is_v ? &tm_v : &tm_k;
#pragma unroll
                    for (int b = 0; b < D / 64; ++b) tma_load_3d(dst + b * (BNK * 128), tm, full, b * 64, j * BNK, bh);
                    if (++st == STAGES) { st = 0; ph ^= 1; }
                }
            }
            if (*abort) {  // drain our own copies before the CTA exits
                if (n_q > 0)
                    for (int t = 0; t < 2; ++t)
                        for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&q_full[t], (n_q - 1) & 1); ++i) {}
                for (uint32_t s = 0; s < (uint32_t)STAGES; ++s) {
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&k_full[s], s < ks ? kp : kp ^ 1); ++i) {}
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&v_full[s], s < vs ? vp : vp ^ 1); ++i) {}
                }
            }
        } else if ((warp == 1 || warp == 2) && lane == 0) {
            // ---------------- score issuers: warp 1 serves tile 0, warp 2 tile 1 ----------------
            const int t = warp - 1;
            const uint32_t idesc_s = idesc_f16(a.is_bf16, /*b_mn_major=*/false, BM, BNK);
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t q_lo = smem_desc_lo(smem_u32(smem + L::Q_OFF + t * L::QTILE), 16);
            const uint32_t k_lo = smem_desc_lo(smem_u32(smem + L::K_OFF), 16);
            const uint32_t s_tmem = tmem_base + t * 128;
            uint32_t stage = 0, phase = 0;
            uint32_t base = 0;  // score blocks of this tile issued in earlier items
            uint32_t n_it = 0;
            bool ok = true;
            for (int r = 0; r < rounds; ++r) {
                int bh, qb;
                if (!item_of_round(r, sc.n_items, sc.n_qb, sc.perm16, bh, qb) || !ok) continue;
                int64_t m0;
                int nkv_t[2], nkv;
                item_extent(a, qb, m0, nkv_t, nkv);
                const int my_nkv = t == 0 ? nkv_t[0] : nkv_t[1];
                ok = mbar_wait(&q_full[t], n_it & 1, abort);
                if (!ok) continue;
                if (t == 1 && n_it == 0) {  // tile 1 starts half a block period late: the two softmaxes take turns on the SFU
                    const long long t_start = clock64();
                    while (clock64() - t_start < kStaggerCycles) {}
                }
                ++n_it;
                for (int j = 0; j < nkv && ok; ++j) {
                    ok = mbar_wait(&k_full[stage], phase, abort);
                    if (!ok) break;
                    if (j < my_nkv) {
                        const uint32_t c = base + j, b = c & 1;
                        // buffer b held S, then P, of this tile's block c - 2: free once that P V has completed
                        if (c >= 2) ok = mbar_wait(&pv_done[t * 2 + b], ((c - 2) >> 1) & 1, abort);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t kb = k_lo + stage * (L::TILE >> 4);
                        const uint32_t d_tmem = s_tmem + b * BNK;
#pragma unroll
                        for (int kk = 0; kk < D / 16; ++kk)
                            tc_mma_f16_halves(d_tmem, q_lo + (((kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4), desc_hi,
                                              kb + (((kk >> 2) * (BNK * 128) + (kk & 3) * 32) >> 4), desc_hi, idesc_s, kk != 0);
                        tc_commit(&s_full[t * 2 + b]);
                    }
                    tc_commit(&k_empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit(&q_empty[t]);  // arrives when every score product of this item has read Q_t
                base += my_nkv;
            }
        } else if (warp == 3 && lane == 0) {
            // ---------------- P V issuer, both tiles in turn ----------------
            const uint32_t idesc_o = idesc_f16(a.is_bf16, /*b_mn_major=*/true, BM, D);
            constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t v_lo = smem_desc_lo(smem_u32(smem + L::V_OFF), BNK * 128);
            uint32_t stage = 0, phase = 0;
            // This thread feeds the tensor core: the loop below is kept instruction for instruction as lean as the one-shot
            // kernel's (measured: testing for the first and the last block of an item inside it, and per-tile completion
            // barriers, cost 10% of the whole kernel).  What an item needs beyond that happens once, outside the loop.
            uint32_t base0 = 0, base1 = 0;  // P blocks consumed per tile in earlier items
            uint32_t n_o = 0;               // items finished
            bool ok = true;
            for (int r = 0; r < rounds; ++r) {
                int bh, qb;
                if (!item_of_round(r, sc.n_items, sc.n_qb, sc.perm16, bh, qb) || !ok) continue;
                int64_t m0;
                int nkv_t[2], nkv;
                item_extent(a, qb, m0, nkv_t, nkv);
                // the first product of an item overwrites O: the previous item's epilogue must have read both accumulators
                ok = mbar_wait(o_empty, (n_o & 1) ^ 1, abort);
                if (!ok) continue;
                for (int j = 0; j < nkv && ok; ++j) {
                    ok = mbar_wait(&v_full[stage], phase, abort);
                    if (!ok) break;
                    const uint32_t vb = v_lo + stage * (L::TILE >> 4);
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (j >= nkv_t[t]) continue;
                        const uint32_t c = (t == 0 ? base0 : base1) + j;
                        ok = mbar_wait(&p_full[t * 2 + (c & 1)], (c >> 1) & 1, abort);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t p_tmem = tmem_base + t * 128 + (c & 1) * BNK;
#pragma unroll
                        for (int kk = 0; kk < BNK / 16; ++kk)  // 16 keys = 8 packed columns of P, 16 rows = 2048 bytes of V
                            tc_mma_f16_ts_halves(tmem_base + 256 + t * 128, p_tmem + kk * 8, vb + kk * (2048 >> 4), desc_hi, idesc_o, (j | kk) != 0);
                        tc_commit(&pv_done[t * 2 + (c & 1)]);
                    }
                    if (!ok) break;
                    tc_commit(&v_empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit(o_full);
                base0 += nkv_t[0];
                base1 += nkv_t[1];
                ++n_o;
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        // ---------------- softmax warpgroups: tile = warpgroup - 1 ----------------
        const int t = (warp >> 2) - 1;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;  // row inside the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem_base + lane_addr + t * 128;
        const uint32_t t_o = tmem_base + lane_addr + 256 + t * 128;
        uint32_t base = 0, n_o = 0;  // score blocks of this tile in earlier items; items finished
        bool ok = true;
        for (int r0 = 0; r0 < rounds; ++r0) {
            int bh, qb;
            if (!item_of_round(r0, sc.n_items, sc.n_qb, sc.perm16, bh, qb) || !ok) continue;
            int64_t m0;
            int nkv_t[2], nkv;
            item_extent(a, qb, m0, nkv_t, nkv);
            const int my_nkv = t == 0 ? nkv_t[0] : nkv_t[1];
            const int seq = (int)a.seq;  // below 2^31 on this path
            const int tile_m0 = (int)m0 + t * BM;
            const int row = tile_m0 + r;
            const int last = a.causal && row < seq ? row : seq - 1;  // last key this row sees
            float m_ref = -INFINITY, l = 0.0f;
            for (int j = 0; j < my_nkv && ok; ++j) {
                const uint32_t c = base + j, b = c & 1;
                ok = mbar_wait(&s_full[t * 2 + b], (c >> 1) & 1, abort);
                if (!ok) break;
                tc_fence_after();
                const int n0 = j * BNK;
                const bool need_mask = (n0 + BNK > seq) || (a.causal && n0 + BNK > tile_m0);
                uint32_t sv[2][32];
#pragma unroll
                for (int c = 0; c < 2; ++c) tmem_ld_32x32(t_s + b * BNK + c * 32, sv[c]);
                tmem_ld_wait();
                float alpha;
                bool rescale;
                softmax_row_lim<2, kPolyPairs>(sv, a.qk_scale, need_mask, last - n0, m_ref, l, alpha, rescale);
                if (j > 0 && __any_sync(0xffffffffu, rescale)) {
                    // O_t must be quiescent: P_t(j-1) V complete (P_t(j) V is not issued before this thread's arrival below)
                    ok = mbar_wait(&pv_done[t * 2 + (b ^ 1)], ((c - 1) >> 1) & 1, abort);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int c0 = 0; c0 < D; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld_32x32(t_o + c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tmem_st_32x32(t_o + c0, v);
                    }
                }
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int e = 2 * i;
                    pk[i] = pack_pair<T>(__uint_as_float(sv[e >> 5][e & 31]), __uint_as_float(sv[e >> 5][(e & 31) + 1]));
                }
                tmem_st_32x32(t_s + b * BNK, pk);
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(&p_full[t * 2 + b]);
            }
            // ---- epilogue: O_t / l; the accumulator is handed back as soon as its last columns are in registers ----
            base += my_nkv;
            ok = ok && mbar_wait(o_full, n_o & 1, abort);  // (every thread of both warpgroups waits and arrives, work or not)
            if (!ok) continue;
            ++n_o;
            tc_fence_after();
            T *o = reinterpret_cast<T *>(a.o) + (int64_t)bh * a.stride_h + (int64_t)row * a.stride_m;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                if (my_nkv > 0) {
                    tmem_ld_32x32(t_o + c0, v);
                    tmem_ld_wait();
                }
                if (c0 + 32 == D) {
                    tc_fence_before();
                    mbar_arrive(o_empty);
                }
                if (my_nkv > 0 && row < seq) {
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __fdiv_rn(__uint_as_float(v[i]), l);
#pragma unroll
                    for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4 *>(o + c0 + 8 * i) = Pack<T>::pack(f + 8 * i);
                }
            }
            if (a.lse && my_nkv > 0 && row < seq) a.lse[(int64_t)bh * a.seq + row] = (m_ref + log2f(l)) * LN2;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort) atomicExch(a.error, 4u);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}
// ---- CUDA-core kernel: any head_dim <= 128, any of the three dtypes, any strides -------------------
// One CTA of 128 threads per (batch*head, 16 query rows): 8 threads share a row and split head_dim.
template <typename T>
__global__ void __launch_bounds__(128) attention_simple_kernel(const T *q, const T *k, const T *v, T *o, float *lse,
                                                              int64_t seq, int d, int64_t stride_h, int64_t stride_m,
                                                              float qk_scale, int causal) {
    constexpr int ROWS = 16, LANES = 8, KV = 32;
    __shared__ float sk[KV][128 + 1], sv[KV][128 + 1];
    const int bh = blockIdx.y;
    const int rl = threadIdx.x / LANES, part = threadIdx.x % LANES;
    const int64_t row = (int64_t)blockIdx.x * ROWS + rl;
    const T *qb = q + (int64_t)bh * stride_h, *kb = k + (int64_t)bh * stride_h, *vb = v + (int64_t)bh * stride_h;
    const bool is_half = sizeof(T) == 2;
    float qr[16], acc[16];  // this thread's slice of head_dim: elements part, part + 8, ...
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int c = part + i * LANES;
        qr[i] = (row < seq && c < d) ? to_f32(qb[row * stride_m + c]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m_i = -INFINITY, l_i = 0.0f;
    const int64_t m_last = (int64_t)blockIdx.x * ROWS + ROWS - 1;
    const int64_t hi = causal ? (m_last + 1 < seq ? m_last + 1 : seq) : seq;
    for (int64_t n0 = 0; n0 < hi; n0 += KV) {
        __syncthreads();
        for (int i = threadIdx.x; i < KV * d; i += blockDim.x) {
            const int rr = i / d, c = i % d;
            const bool okr = n0 + rr < seq;
            sk[rr][c] = okr ? to_f32(kb[(n0 + rr) * stride_m + c]) : 0.0f;
            sv[rr][c] = okr ? to_f32(vb[(n0 + rr) * stride_m + c]) : 0.0f;
        }
        __syncthreads();
        float s[KV];
        float mx = -INFINITY;
#pragma unroll 4
        for (int jj = 0; jj < KV; ++jj) {
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int c = part + i * LANES;
                if (c < d) dot = fmaf(qr[i], sk[jj][c], dot);
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            const int64_t col = n0 + jj;
            float sc = dot * qk_scale;
            if (col >= seq || (causal && col > row)) sc = -INFINITY;
            s[jj] = sc;
            mx = fmaxf(mx, sc);
        }
        const float m_new = fmaxf(m_i, mx);
        const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
        const float alpha = m_i == -INFINITY ? 0.0f : exp2f(m_i - m_safe);
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] *= alpha;
#pragma unroll 4
        for (int jj = 0; jj < KV; ++jj) {
            const float p = exp2f(s[jj] - m_safe);
            sum += p;
            const float pr = is_half ? to_f32(from_f32<T>(p)) : p;  // P rounded to the input type
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int c = part + i * LANES;
                if (c < d) acc[i] = fmaf(pr, sv[jj][c], acc[i]);
            }
        }
        l_i = l_i * alpha + sum;
        m_i = m_new;
    }
    if (row < seq) {
        T *ob = o + (int64_t)bh * stride_h + row * stride_m;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int c = part + i * LANES;
            if (c < d) ob[c] = from_f32<T>(__fdiv_rn(acc[i], l_i));
        }
        if (lse && part == 0) lse[(int64_t)bh * seq + row] = (m_i + log2f(l_i)) * LN2;
    }
}

// 0: two 128-row query tiles per CTA, 128-key blocks, P in TMEM; 1, 2: one tile, P through shared memory, 4- or 3-deep
// K/V ring; 3: two tiles, 64-key blocks, one CTA per 256 query rows; 4: the same as persistent CTAs over a static schedule
constexpr int ATTN_VARIANTS = 5;

// Tensor maps over [bh, seq, D] with boxes of 64 values x 128 rows (64 rows for K and V when KV_ROWS is 64),
// then the launch.  TILES = query tiles of 128 rows per CTA.
template <typename T, int D, int STAGES, int TILES, int KV_ROWS = 128>
int launch_tc(const void *q, const void *k, const void *v, const AttnArgs &args, int64_t bh, cudaStream_t st) {
    char err[256];
    CUtensorMap tq, tk, tv;
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)args.seq, (uint64_t)bh};
    const uint64_t strides[2] = {(uint64_t)args.stride_m * 2, (uint64_t)args.stride_h * 2};
    const uint32_t box[3] = {64, BM, 1}, kv_box[3] = {64, KV_ROWS, 1};
    if (!make_tensor_map(&tq, q, args.is_bf16, 3, dims, strides, box, err, sizeof(err)) ||
        !make_tensor_map(&tk, k, args.is_bf16, 3, dims, strides, kv_box, err, sizeof(err)) ||
        !make_tensor_map(&tv, v, args.is_bf16, 3, dims, strides, kv_box, err, sizeof(err)))
        return fail(ENC_ERR_LAUNCH, "enc_attention_fwd: %s", err);
    auto kern = TILES == 1 ? attention_tc_kernel<T, D, STAGES> : KV_ROWS == 64 ? attention_ts64_kernel<T, D, STAGES> : attention_ts_kernel<T, D, STAGES>;
    const int smem = (TILES == 1 ? AttnSmem<D, STAGES>::TOTAL : KV_ROWS == 64 ? AttnSmem64<D, STAGES>::TOTAL : AttnSmemTs<D, STAGES>::TOTAL) + 1024;
    const int threads = TILES == 2 ? kThreads2 : kThreads;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_attention_fwd: cannot opt in to %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    dim3 grid((unsigned)cdiv(args.seq, TILES * BM), (unsigned)bh);
    kern<<<grid, threads, smem, st>>>(tq, tk, tv, args);
    return check_launch("enc_attention_fwd");
}

// Query-block order inside a slice for the persistent kernel's zigzag schedule (see attention_p64_kernel): the two
// items a CTA gets in rounds 2m and 2m+1 are k1 = 2mG + c and k2 = (2m+1)G + G-1-c, so their positions inside a slice
// satisfy q1 + q2 = (4m+2)G - 1 (mod n), which is the same s for every m when 4G is a multiple of n.  Positions that
// pair up get query blocks that add up to n-1, i.e. causal key-block counts that add up to a constant.
uint64_t balance_perm16(int G, int n) {
    uint64_t identity = 0;
    for (int q = 0; q < 16; ++q) identity |= (uint64_t)q << (4 * q);
    if (n > 16 || n < 2) return identity;
    const int s = (int)(((2LL * G - 1) % n + n) % n);
    int assigned[16];
    bool used[16] = {};
    for (int q = 0; q < n; ++q) assigned[q] = -1;
    int lo = 0;
    for (int q = 0; q < n; ++q) {
        const int q2 = ((s - q) % n + n) % n;
        if (assigned[q] >= 0 || q2 == q) continue;
        assigned[q] = lo;
        assigned[q2] = n - 1 - lo;
        used[lo] = used[n - 1 - lo] = true;
        ++lo;
    }
    int next = 0;
    for (int q = 0; q < n; ++q) {  // positions paired with themselves take the values that are left (the middle ones)
        if (assigned[q] >= 0) continue;
        while (used[next]) ++next;
        assigned[q] = next;
        used[next] = true;
    }
    uint64_t perm = 0;
    for (int q = 0; q < n; ++q) perm |= (uint64_t)assigned[q] << (4 * q);
    return perm;
}

template <typename T, int D, int STAGES>
int launch_persistent(const void *q, const void *k, const void *v, const AttnArgs &args, int64_t bh, cudaStream_t st) {
    char err[256];
    CUtensorMap tq, tk, tv;
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)args.seq, (uint64_t)bh};
    const uint64_t strides[2] = {(uint64_t)args.stride_m * 2, (uint64_t)args.stride_h * 2};
    const uint32_t box[3] = {64, BM, 1}, kv_box[3] = {64, BN64, 1};
    if (!make_tensor_map(&tq, q, args.is_bf16, 3, dims, strides, box, err, sizeof(err)) ||
        !make_tensor_map(&tk, k, args.is_bf16, 3, dims, strides, kv_box, err, sizeof(err)) ||
        !make_tensor_map(&tv, v, args.is_bf16, 3, dims, strides, kv_box, err, sizeof(err)))
        return fail(ENC_ERR_LAUNCH, "enc_attention_fwd: %s", err);
    auto kern = attention_p64_kernel<T, D, STAGES>;
    const int smem = AttnSmemP<D, STAGES>::TOTAL + 1024;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_attention_fwd: cannot opt in to %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    Sched sc;
    sc.n_qb = (int)cdiv(args.seq, 2 * BM);
    const int64_t items = (int64_t)sc.n_qb * bh;
    if (items > 0x7fffffffLL) return fail(ENC_ERR_UNSUPPORTED, "enc_attention_fwd: more than 2^31-1 work items");
    sc.n_items = (int)items;
    int grid = device_props().sm_count;
    sc.perm16 = balance_perm16(grid, 0);  // identity
    if (args.causal && sc.n_qb >= 2 && sc.n_qb <= 16 && items > grid) {
        // the pairing needs 4 * grid to be a multiple of n_qb: give up a few SMs (at most 5%) for it when necessary
        int g = grid;
        while (g > 0 && (4LL * g) % sc.n_qb != 0) --g;
        if (g * 20 >= grid * 19) {
            grid = g;
            sc.perm16 = balance_perm16(grid, sc.n_qb);
        }
    }
    if (grid > items) grid = (int)items;
    kern<<<(unsigned)grid, kThreads2, smem, st>>>(tq, tk, tv, args, sc);
    return check_launch("enc_attention_fwd");
}

template <typename T>
int launch_attention(const void *q, const void *k, const void *v, AttnArgs args, int64_t bh, int64_t d, int variant,
                     cudaStream_t st) {
    const bool tc = sizeof(T) == 2 && (d == 64 || d == 128) && aligned16(q) && aligned16(k) && aligned16(v) &&
                    aligned16(args.o) && args.stride_m % 8 == 0 && args.stride_h % 8 == 0 && bh <= 65535 &&
                    args.seq < (1LL << 31);
    if (!tc) {
        if (bh > 65535) return fail(ENC_ERR_UNSUPPORTED, "enc_attention_fwd: more than 65535 (batch, head) slices");
        dim3 grid((unsigned)cdiv(args.seq, 16), (unsigned)bh);
        attention_simple_kernel<T><<<grid, 128, 0, st>>>((const T *)q, (const T *)k, (const T *)v, (T *)args.o, args.lse,
                                                         args.seq, (int)d, args.stride_h, args.stride_m, args.qk_scale,
                                                         args.causal);
        return check_launch("enc_attention_fwd");
    }
    args.error = device_error_word();
    if (!args.error) return fail(ENC_ERR_NO_MEMORY, "enc_attention_fwd: cannot allocate the device status word");
    if constexpr (sizeof(T) == 2) {
        if (variant < 0) {
            // Two tiles per CTA once there are two tiles.  One-shot grid (variant 3) or persistent CTAs (variant 4), as measured
            // on B200 (bf16/f16, D = 128 and 64, sequences 512 to 16384).  The persistent kernel saves the per-item set-up and
            // balances causal work statically, but its inner loops still run about 5% slower than the one-shot kernel's, so it
            // wins where items are short or uneven: causal launches up to 4096 keys (+3% at [8,32,4096,128], +9% at 2048, +13%
            // at 512, +27-32% at [1,16,4096,D], where the hardware's dispatch order cannot balance 256 uneven CTAs over 148
            // SMs) and non-causal launches up to 2048 keys (+1% to +13%).  It loses with long non-causal items (-5% at 4096
            // keys, -14% at 16384), beyond 4096 keys causal (its balancing permutation covers 16 query blocks), and whenever
            // there is at most one item per SM.
            const int64_t items = cdiv(args.seq, 2 * BM) * bh, sms = device_props().sm_count;
            const bool persistent = items > sms && args.seq <= (args.causal ? 4096 : 2048);
            variant = args.seq <= BM ? 1 : persistent ? 4 : 3;
        }
        if (variant == 4) return d == 128 ? launch_persistent<T, 128, 5>(q, k, v, args, bh, st) : launch_persistent<T, 64, 6>(q, k, v, args, bh, st);
        if (d == 128) {
            if (variant == 0) return launch_tc<T, 128, 5, 2>(q, k, v, args, bh, st);
            if (variant == 3) return launch_tc<T, 128, 5, 2, 64>(q, k, v, args, bh, st);
            return variant == 2 ? launch_tc<T, 128, 3, 1>(q, k, v, args, bh, st) : launch_tc<T, 128, 4, 1>(q, k, v, args, bh, st);
        }
        if (variant == 0) return launch_tc<T, 64, 8, 2>(q, k, v, args, bh, st);
        if (variant == 3) return launch_tc<T, 64, 6, 2, 64>(q, k, v, args, bh, st);
        return variant == 2 ? launch_tc<T, 64, 3, 1>(q, k, v, args, bh, st) : launch_tc<T, 64, 4, 1>(q, k, v, args, bh, st);
    }
    return fail(ENC_ERR_UNSUPPORTED, "enc_attention_fwd: unreachable");
}

}  // namespace

int attention_variants() { return ATTN_VARIANTS; }
void attention_variant_info(int v, char *out, size_t n) {
    if (v == 0) snprintf(out, n, "block_m=256 (two 128-row tiles, one softmax warpgroup each) block_n=128 tcgen05 S/P/O in TMEM");
    else if (v == 3) snprintf(out, n, "block_m=256 (two 128-row tiles) block_n=64 tcgen05 S/P/O in TMEM, score products issued one block ahead");
    else if (v == 4) snprintf(out, n, "block_m=256 block_n=64 as variant 3, persistent CTAs (one per SM) over a static balanced schedule");
    else snprintf(out, n, "block_m=128 block_n=128 kv_stages=%d tcgen05 S/O in TMEM, P through shared memory", v == 2 ? 3 : 4);
}

}  // namespace enc

extern "C" int enc_attention_fwd(const void *q, const void *k, const void *v, void *o, float *lse, int64_t bh,
                                 int64_t seq, int64_t head_dim, int64_t stride_h, int64_t stride_m, float sm_scale,
                                 int causal, int dtype, int variant, void *stream) {
    ENC_PROLOGUE();
    if (bh < 0 || seq < 0 || head_dim <= 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_attention_fwd: bad shape");
    if (bh == 0 || seq == 0) return ENC_OK;
    if (!q || !k || !v || !o) return enc::fail(ENC_ERR_BAD_ARG, "enc_attention_fwd: NULL tensor");
    if (head_dim > 128) return enc::fail(ENC_ERR_UNSUPPORTED, "enc_attention_fwd: head_dim %lld > 128", (long long)head_dim);
    if (stride_m < head_dim) return enc::fail(ENC_ERR_BAD_ARG, "enc_attention_fwd: row stride smaller than head_dim");
    if (variant >= enc::ATTN_VARIANTS) return enc::fail(ENC_ERR_BAD_ARG, "enc_attention_fwd: variant %d out of range", variant);
    enc::AttnArgs args{o, lse, seq, stride_h, stride_m, sm_scale * enc::LOG2E, causal ? 1 : 0, dtype == ENC_BF16 ? 1 : 0, nullptr};
    cudaStream_t st = enc::as_stream(stream);
    switch (dtype) {
        case ENC_F16: return enc::launch_attention<__half>(q, k, v, args, bh, head_dim, variant, st);
        case ENC_BF16: return enc::launch_attention<__nv_bfloat16>(q, k, v, args, bh, head_dim, variant, st);
        case ENC_F32: return enc::launch_attention<float>(q, k, v, args, bh, head_dim, variant, st);
        default: return enc::fail(ENC_ERR_BAD_ARG, "enc_attention_fwd: dtype %d is not float16, bfloat16 or float32", dtype);
    }
}
