// Row softmax, LayerNorm and RMSNorm for sm_100a.
//
// All three are HBM-bound: one read and one write of the matrix.  A row is loaded ONCE with
// 128-bit streaming loads into registers (up to 32 float values per thread), reduced with warp
// shuffles plus one shared-memory exchange when a row spans several warps, and written back with
// 128-bit stores.  Statistics are float32; the LayerNorm variance comes from one pass over the registers
// (sum and sum of squares), with the reference's centred second pass, again from the registers, for rows
// whose mean is large against their spread, so nothing is re-read.  Rows wider than the register budget
// take a three-pass kernel that re-reads the row through L2.
//
// The formulas are the reference kernels' (examples/02_softmax.py:15-24, examples/03_layernorm.py:15-42,
// examples/06_rmsnorm.py:15-24): max-subtracted softmax, biased variance, 1/sqrt(var+eps).
// At B200's ratio of HBM bandwidth to FP32 issue rate a bf16 element has a budget of about twenty
// lane-instructions, so the per-element work is kept short: fused multiply-adds where the reference
// rounds twice, exp as ex2.approx of a pre-scaled argument, one reciprocal per row instead of a
// division per element.  Each of these moves a result by a few float32 ulps, far inside the
// tolerances the results are held to (1e-5 for float32 outputs).
// A leaner form was measured on LayerNorm bf16 [16384, 4096] (then 17 executed instructions per element, 5.83 TB/s;
// 13.7 and 5.92 TB/s with the fast path below) and
// rejected: looping CTAs one row wide that convert weight and bias once and keep the next rows' loads in flight in
// registers (about 7 instructions per element, but 8 to 16 warps per SM cannot hide the per-row reduction chain:
// 5.05 TB/s at best).  What did pay is a path without bounds tests for rows that fill their threads exactly, once
// the registers of those instantiations were capped (row_max_regs below).
// For the short rows of softmax float32 [4096, 1024] (one wave of CTAs, 6.7 us) a warp that owns two rows and issues both
// rows' loads up front was measured as well: 4.47 against 5.07 TB/s.  The loads of a wave already return spread over
// the 2.6 us the memory system needs for them, so the arithmetic of early rows overlaps the arrival of late ones as it
// is, and halving the number of warps only lengthens the arithmetic.
#include <map>
#include <mutex>
#include <tuple>

#include "sm100.cuh"

namespace enc {
namespace {

constexpr int MAX_WARPS = 32;

struct RowArgs {
    const void *x;
    void *y;
    const void *w;
    const void *b;
    float *mean;
    float *rstd;
    int64_t rows, cols, stride_x, stride_y;
    float eps;
    int tpr;  // threads per row (power of two, 32..512)
};

enum { OP_SOFTMAX = 0, OP_LAYERNORM = 1, OP_RMSNORM = 2 };
// Packed f32x2 instructions, as a bit mask: 1 = LayerNorm sums, 2 = LayerNorm output, 4 = RMSNorm (both passes).
// Measured at bf16 [16384, 4096]: 2 and 4 gain 1-2%, 1 loses 3% (the pair moves cost more than the adds save).
constexpr int ROW_PACKED_MASK = 2 | 4;

// Reduction over the `tpr` threads that share a row.  `slot` is a per-call shared array so that
// consecutive reductions need one barrier each.
template <bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, int tpr, float *slot) {
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    if (tpr > 32) {
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) slot[warp] = v;
        __syncthreads();
        const int wpr = tpr >> 5;                     // warps per row
        const int first = (warp / wpr) * wpr;         // first warp of this row group
        float r = slot[first];
        for (int i = 1; i < wpr; ++i) r = IS_MAX ? fmaxf(r, slot[first + i]) : r + slot[first + i];
        v = r;
    }
    return v;
}

// Two sums at once over the threads of a row: one barrier instead of two.
__device__ __forceinline__ void group_sum2(float &x, float &y, int tpr, float *slot_x, float *slot_y) {
    x = warp_sum(x);
    y = warp_sum(y);
    if (tpr > 32) {
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) {
            slot_x[warp] = x;
            slot_y[warp] = y;
        }
        __syncthreads();
        const int wpr = tpr >> 5;
        const int first = (warp / wpr) * wpr;
        float rx = slot_x[first], ry = slot_y[first];
        for (int i = 1; i < wpr; ++i) {
            rx += slot_x[first + i];
            ry += slot_y[first + i];
        }
        x = rx;
        y = ry;
    }
}

// A row lives in registers as V raw 16-byte vectors per thread (float16/bfloat16 stay packed, which
// halves the register cost and lets one warp hold a 4096-wide row); every pass unpacks to float32
// on the fly.
template <typename T, int V> union RowRegs {
    uint4 v[V];
    T e[V * Pack<T>::N];
    __device__ RowRegs() {}
};

// Statistics and output of one row held in `x`.  WB = true: weight/bias vectors are already in the
// registers `wreg`/`breg` (persistent CTAs); otherwise they are fetched from global memory (L2-resident).
// Every thread of the CTA must call this the same number of times (it contains CTA barriers).
// FULL = true: the row is exactly tpr * V vectors wide, so no vector of any thread is cut or past the end and every
// bounds test disappears (they cost three to four of the seventeen instructions per element).
template <typename T, int V, bool VEC, int OP, bool WB, bool FULL = false>
__device__ __forceinline__ void process_row(const RowRegs<T, V> &x, const RowArgs &a, int tpr, int t, int64_t row,
                                            bool live, float *red0, float *red1, float *red2, const uint4 *wreg,
                                            const uint4 *breg) {
    constexpr int NV = Pack<T>::N;
    const float fill = OP == OP_SOFTMAX ? -INFINITY : 0.0f;
    // value (j, e) as float, `fill` beyond the row
    const int cols = (int)a.cols;
    auto get = [&](int j, float *f) {
        const int c0 = (j * tpr + t) * NV;
        if (VEC) {
            if (FULL || c0 < cols) {
                Pack<T>::unpack(x.v[j], f);
            } else {
#pragma unroll
                for (int e = 0; e < NV; ++e) f[e] = fill;
            }
        } else {
#pragma unroll
            for (int e = 0; e < NV; ++e) f[e] = (c0 + e < cols) ? to_f32(x.e[j * NV + e]) : fill;
        }
    };

    constexpr float LOG2E = 1.4426950408889634f;
    // Softmax needs every exponential twice (row sum, output).  They are kept in registers (as float32) when a thread
    // holds at most 64 elements of the row: always for float32 rows, and for 16-bit rows once the row is spread over
    // twice the minimum number of threads (the launcher's default for wide 16-bit rows); otherwise they are recomputed.
    constexpr bool KEEP_EXP = OP == OP_SOFTMAX && V * NV <= 64;
    float ex[KEEP_EXP ? V * NV : 1];
    float s0 = 1.0f, s1 = 0.0f;  // softmax: -max*log2e, 1/sum.  layernorm: rstd, -mean*rstd.  rmsnorm: rstd.
    if (OP == OP_SOFTMAX) {
        float m = -INFINITY;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            float f[NV];
            get(j, f);
#pragma unroll
            for (int e = 0; e < NV; ++e) m = fmaxf(m, f[e]);
        }
        m = group_reduce<true>(m, tpr, red0);
        const float nm = -m * LOG2E;  // exp(x - m) = 2^(x*log2e - m*log2e)
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            float f[NV];
            get(j, f);
#pragma unroll
            for (int e = 0; e < NV; ++e) {
                const float p = fast_exp2(fmaf(f[e], LOG2E, nm));
                s += p;
                if (KEEP_EXP) ex[j * NV + e] = p;  // float32 rows: the exponentials take the registers the row leaves
            }
        }
        s0 = nm;
        s1 = __fdiv_rn(1.0f, group_reduce<false>(s, tpr, red1));
    } else if (OP == OP_LAYERNORM) {
        // One pass gives sum and sum of squares (fill values are zero, so they do not disturb either);
        // var = E[x^2] - mean^2 is accurate to a few ulps as long as the mean is not large against the
        // spread.  When it is (mean^2 > 16 var: cancellation would cost more than 1e-6 of relative
        // accuracy), the variance is recomputed from the registers in the centred form the reference
        // uses.  The choice is made for the whole CTA because the reductions contain CTA barriers.
        float s = 0.0f, q = 0.0f;
        if (ROW_PACKED_MASK & 1) {  // two values per add / fma (even and odd elements form two chains)
            uint64_t s2 = f2_pack(0.0f, 0.0f), q2 = s2;
#pragma unroll
            for (int j = 0; j < V; ++j) {
                float f[NV];
                get(j, f);
#pragma unroll
                for (int e = 0; e < NV; e += 2) {
                    const uint64_t p = f2_pack(f[e], f[e + 1]);
                    s2 = f2_add(s2, p);
                    q2 = f2_fma(p, p, q2);
                }
            }
            float lo, hi;
            f2_unpack(s2, lo, hi);
            s = lo + hi;
            f2_unpack(q2, lo, hi);
            q = lo + hi;
        } else {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                float f[NV];
                get(j, f);
#pragma unroll
                for (int e = 0; e < NV; ++e) {
                    s += f[e];
                    q = fmaf(f[e], f[e], q);
                }
            }
        }
        const float n = (float)a.cols;
        group_sum2(s, q, tpr, red0, red1);
        const float mean = __fdiv_rn(s, n);
        float var = fmaf(-mean, mean, __fdiv_rn(q, n));
        const bool ill = !(mean * mean <= 16.0f * var);  // also catches var <= 0 and NaN
        // (a CTA that holds a single row already agrees on `ill` and needs no vote)
        if ((int)blockDim.x == tpr ? ill : (bool)__syncthreads_or(ill)) {
            float qc = 0.0f;
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const int c0 = (j * tpr + t) * NV;
                if (VEC && !FULL && c0 >= cols) continue;  // a vector is inside the row or entirely past it
                float f[NV];
                get(j, f);
#pragma unroll
                for (int e = 0; e < NV; ++e) {
                    const float d = (VEC || c0 + e < cols) ? f[e] - mean : 0.0f;
                    qc = fmaf(d, d, qc);
                }
            }
            var = __fdiv_rn(group_reduce<false>(qc, tpr, red2), n);
        }
        const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, a.eps)));
        s0 = rstd;
        s1 = -mean * rstd;  // (x - mean) * rstd = x*rstd - mean*rstd
        if (live && t == 0) {
            if (a.mean) a.mean[row] = mean;
            if (a.rstd) a.rstd[row] = rstd;
        }
    } else {
        float q = 0.0f;
        if (ROW_PACKED_MASK & 4) {
            uint64_t q2 = f2_pack(0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < V; ++j) {
                float f[NV];
                get(j, f);
#pragma unroll
                for (int e = 0; e < NV; e += 2) {
                    const uint64_t p = f2_pack(f[e], f[e + 1]);
                    q2 = f2_fma(p, p, q2);
                }
            }
            float lo, hi;
            f2_unpack(q2, lo, hi);
            q = lo + hi;
        } else {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                float f[NV];
                get(j, f);
#pragma unroll
                for (int e = 0; e < NV; ++e) q = fmaf(f[e], f[e], q);
            }
        }
        const float ms = __fdiv_rn(group_reduce<false>(q, tpr, red0), (float)a.cols);
        s0 = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, a.eps)));
    }
    if (!live) return;

    T *yr = reinterpret_cast<T *>(a.y) + row * a.stride_y;
    const T *wr = reinterpret_cast<const T *>(a.w);
    const T *br = reinterpret_cast<const T *>(a.b);
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int c0 = (j * tpr + t) * NV;
        if (!FULL && c0 >= cols) continue;
        float f[NV], wv[NV], bv[NV];
        get(j, f);
        if (OP != OP_SOFTMAX) {
            if (WB) {
                Pack<T>::unpack(wreg[j], wv);
                if (OP == OP_LAYERNORM) Pack<T>::unpack(breg[j], bv);
            } else if (VEC) {
                Pack<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(wr + c0)), wv);
                if (OP == OP_LAYERNORM) Pack<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(br + c0)), bv);
            } else {
#pragma unroll
                for (int e = 0; e < NV; ++e) {
                    const bool ok = c0 + e < cols;
                    wv[e] = ok ? to_f32(wr[c0 + e]) : 0.0f;
                    if (OP == OP_LAYERNORM) bv[e] = ok ? to_f32(br[c0 + e]) : 0.0f;
                }
            }
        }
        float o[NV];
        if ((OP == OP_LAYERNORM && (ROW_PACKED_MASK & 2)) || (OP == OP_RMSNORM && (ROW_PACKED_MASK & 4))) {
            const uint64_t s02 = f2_pack(s0, s0), s12 = f2_pack(s1, s1);
#pragma unroll
            for (int e = 0; e < NV; e += 2) {
                const uint64_t p = f2_pack(f[e], f[e + 1]), w2 = f2_pack(wv[e], wv[e + 1]);
                const uint64_t r = OP == OP_LAYERNORM ? f2_fma(f2_fma(p, s02, s12), w2, f2_pack(bv[e], bv[e + 1])) : f2_mul(f2_mul(p, s02), w2);
                f2_unpack(r, o[e], o[e + 1]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < NV; ++e) {
                if (OP == OP_SOFTMAX) o[e] = (KEEP_EXP ? ex[j * NV + e] : fast_exp2(fmaf(f[e], LOG2E, s0))) * s1;
                else if (OP == OP_LAYERNORM) o[e] = fmaf(fmaf(f[e], s0, s1), wv[e], bv[e]);
                else o[e] = (f[e] * s0) * wv[e];
            }
        }
        if (VEC) {
            st_stream(yr + c0, Pack<T>::pack(o));
        } else {
#pragma unroll
            for (int e = 0; e < NV; ++e)
                if (c0 + e < cols) yr[c0 + e] = from_f32<T>(o[e]);
        }
    }
}

// One CTA per group of blockDim/tpr rows; the rows go straight from global memory to registers.
// Register cap of an instantiation.  With the fast path above the compiler would keep a whole unpacked row in registers
// (104 per thread for LayerNorm bf16, 8 vectors), which costs more in resident warps than the saved unpacking brings
// back, and capped at 64 it spills.  Measured per cap (TB/s, default variants): LayerNorm bf16 [16384, 4096]: 4.58 at
// 64, 5.40 at 72, 5.92 at 80, 5.76 at 96, 5.31 uncapped (5.81 before the fast path); softmax float32 [4096, 1024]:
// 5.03, 5.28, 5.17, 5.16, 5.18 (5.06 before).  Rows of at most 4 vectors per thread need no cap, and 16 vectors (64
// registers of packed row data) need all 128.
template <typename T, int V, int OP> constexpr int row_max_regs() {
    if (V == 4 && OP == OP_RMSNORM && sizeof(T) == 2) return 56;  // RMSNorm bf16 [16384, 4096]: 6.67 against 6.50 TB/s uncapped (6.63 at 48, 5.04 at 40)
    if (V != 8) return 128;
    if (OP == OP_SOFTMAX) return sizeof(T) == 4 ? 72 : 80;
    // LayerNorm fp16 [4096, 4096]: 4.73 at 88 against 4.48 at 80 (bf16 [16384, 4096] the same at both); RMSNorm fp32
    // [4096, 4096]: 6.29 against 6.19; LayerNorm fp32: 5.92 against 5.97
    return (OP == OP_LAYERNORM) == (sizeof(T) == 2) ? 88 : 80;
}

template <typename T, int V, bool VEC, int OP>
__global__ void __maxnreg__((row_max_regs<T, V, OP>())) row_kernel(RowArgs a) {
    constexpr int NV = Pack<T>::N;
    __shared__ float red0[MAX_WARPS], red1[MAX_WARPS], red2[MAX_WARPS];
    const int tpr = a.tpr;
    const int t = threadIdx.x & (tpr - 1);
    const int64_t rows_per_cta = blockDim.x / tpr;
    const int64_t row = (int64_t)blockIdx.x * rows_per_cta + threadIdx.x / tpr;
    const bool live = row < a.rows;
    const T *xr = reinterpret_cast<const T *>(a.x) + (live ? row : 0) * a.stride_x;
    // (Asking L2 for the whole input with bulk prefetches before the dependency wait, from the first CTA of every SM, was
    // measured on the small shapes it could help and lost 5-10%: the CTAs that issue the prefetches start their own
    // rows late.)
    grid_dependency_wait();  // launched with launch_overlapped(): nothing above touches global memory

    RowRegs<T, V> x;
    const int cols = (int)a.cols;
    if (VEC && cols == tpr * (V * NV)) {  // every vector of every thread is inside the row: no bounds tests anywhere
#pragma unroll
        for (int j = 0; j < V; ++j) x.v[j] = ld_stream(xr + (j * tpr + t) * NV);
        process_row<T, V, VEC, OP, false, true>(x, a, tpr, t, row, live, red0, red1, red2, nullptr, nullptr);
        return;
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int c0 = (j * tpr + t) * NV;
        if (VEC) {
            if (c0 < cols) x.v[j] = ld_stream(xr + c0);
        } else {
#pragma unroll
            for (int e = 0; e < NV; ++e)
                if (c0 + e < cols) x.e[j * NV + e] = xr[c0 + e];
        }
    }
    process_row<T, V, VEC, OP, false>(x, a, tpr, t, row, live, red0, red1, red2, nullptr, nullptr);
}

// Persistent CTAs fed by the bulk-copy engine.  Each CTA owns a ring of STAGES buffers in shared
// memory; one elected thread keeps the ring full with cp.async.bulk row copies (completion counted in
// bytes on the stage's mbarrier), the CTA's threads pull a stage into registers, hand the buffer back,
// and compute and store from registers.  The bytes in flight per SM are set by the ring depth, not by
// how many registers or warps the arithmetic needs, which is what a kernel with two CTA-wide
// reductions per row (LayerNorm) needs to stay at HBM speed.  Weight and bias stay in registers across
// rows.  Rows must be 16-byte aligned and a whole number of 16-byte vectors (the VEC conditions).
struct PipeArgs {
    RowArgs r;
    int stages;
    unsigned *error;
};

template <typename T, int V, int OP>
__global__ void __launch_bounds__(512, 1) row_pipe_kernel(PipeArgs p) {
    using namespace sm100;
    constexpr int NV = Pack<T>::N;
    extern __shared__ __align__(128) uint8_t pipe_smem[];
    __shared__ float red0[MAX_WARPS], red1[MAX_WARPS], red2[MAX_WARPS];
    __shared__ uint64_t full[16];
    const RowArgs &a = p.r;
    const int tpr = a.tpr, S = p.stages;
    const int t = threadIdx.x & (tpr - 1), g = threadIdx.x / tpr;
    const int R = blockDim.x / tpr;  // rows per stage
    const uint32_t row_bytes = (uint32_t)(a.cols * sizeof(T));
    const int64_t nblocks = (a.rows + R - 1) / R;
    const T *xg = reinterpret_cast<const T *>(a.x);

    auto fill_stage = [&](int s, int64_t blk) {  // thread 0 only
        const int64_t r0 = blk * R;
        const int live_rows = a.rows - r0 < R ? (int)(a.rows - r0) : R;
        mbar_expect_tx(&full[s], row_bytes * live_rows);
        for (int i = 0; i < live_rows; ++i) {
            const uint32_t dst = smem_u32(pipe_smem + ((size_t)s * R + i) * row_bytes);
            asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dst), "l"(xg + (r0 + i) * a.stride_x), "r"(row_bytes), "r"(smem_u32(&full[s])) : "memory");
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            const int64_t blk = blockIdx.x + (int64_t)s * gridDim.x;
            if (blk < nblocks) fill_stage(s, blk);
        }
    }
    // weight / bias for this thread's columns, kept for every row
    uint4 wreg[V], breg[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int64_t c0 = ((int64_t)j * tpr + t) * NV;
        wreg[j] = breg[j] = make_uint4(0, 0, 0, 0);
        if (OP != OP_SOFTMAX && c0 < a.cols) {
            wreg[j] = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.w) + c0));
            if (OP == OP_LAYERNORM) breg[j] = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.b) + c0));
        }
    }

    int s = 0;
    uint32_t parity = 0;
    for (int64_t blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
        // bounded wait for the stage; on expiry raise the error word and carry on with what is there
        bool ready = false;
        for (uint32_t i = 0; i < (1u << 20) && !ready; ++i) ready = mbar_try_wait(&full[s], parity);
        if (!ready) atomicExch(p.error, 3u);
        const int64_t row = blk * R + g;
        const bool live = row < a.rows;
        RowRegs<T, V> x;
        const uint8_t *src = pipe_smem + ((size_t)s * R + g) * row_bytes;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const int64_t c0 = ((int64_t)j * tpr + t) * NV;
            if (c0 < a.cols) x.v[j] = *reinterpret_cast<const uint4 *>(src + c0 * sizeof(T));
        }
        __syncthreads();  // every thread has taken its part of the stage
        if (threadIdx.x == 0) {
            const int64_t next = blk + (int64_t)S * gridDim.x;
            if (next < nblocks) {
                fence_proxy_async();  // order the reads above before the bulk copy overwrites the buffer
                fill_stage(s, next);
            }
        }
        process_row<T, V, true, OP, true>(x, a, tpr, t, live ? row : 0, live, red0, red1, red2, wreg, breg);
        if (++s == S) { s = 0; parity ^= 1; }
    }
}

// Rows too wide for registers: one 1024-thread CTA per row, three passes through L2.
template <bool IS_MAX> __device__ float cta_reduce(float v, float *slot) {
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    __syncthreads();  // slot may still be read from the previous reduction
    if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = slot[0];
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) r = IS_MAX ? fmaxf(r, slot[i]) : r + slot[i];
    return r;
}

template <typename T, int OP>
__global__ void __launch_bounds__(1024) row_kernel_wide(RowArgs a) {
    __shared__ float red[MAX_WARPS];
    const int64_t row = blockIdx.x;
    const T *xr = reinterpret_cast<const T *>(a.x) + row * a.stride_x;
    T *yr = reinterpret_cast<T *>(a.y) + row * a.stride_y;
    const T *wr = reinterpret_cast<const T *>(a.w);
    const T *br = reinterpret_cast<const T *>(a.b);
    const float n = (float)a.cols;
    if (OP == OP_SOFTMAX) {
        float m = -INFINITY;
        for (int64_t c = threadIdx.x; c < a.cols; c += blockDim.x) m = fmaxf(m, to_f32(xr[c]));
        m = cta_reduce<true>(m, red);
        float s = 0.0f;
        for (int64_t c = threadIdx.x; c < a.cols; c += blockDim.x) s += expf(__fsub_rn(to_f32(xr[c]), m));
        s = cta_reduce<false>(s, red);
        for (int64_t c = threadIdx.x; c < a.cols; c += blockDim.x)
            yr[c] = from_f32<T>(__fdiv_rn(expf(__fsub_rn(to_f32(xr[c]), m)), s));
    } else if (OP == OP_LAYERNORM) {
        float s = 0.0f;
        for (int64_t c = threadIdx.x; c < a.cols; c += blockDim.x) s += to_f32(xr[c]);
        const float mean = __fdiv_rn(cta_reduce<false>(s, red), n);
        float q = 0.0f;
        for (int64_t c = threadIdx.x; c < a.cols; c += blockDim.x) {
            const float d = __fsub_rn(to_f32(xr[c]), mean);
            q = __fadd_rn(q, __fmul_rn(d, d));
        }
        const float var = __fdiv_rn(cta_reduce<false>(q, red), n);
        const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, a.eps)));
        if (threadIdx.x == 0) {
            if (a.mean) a.mean[row] = mean;
            if (a.rstd) a.rstd[row] = rstd;
        }
        for (int64_t c = threadIdx.x; c < a.cols; c += blockDim.x) {
            const float d = __fsub_rn(to_f32(xr[c]), mean);
            yr[c] = from_f32<T>(__fadd_rn(__fmul_rn(__fmul_rn(d, rstd), to_f32(wr[c])), to_f32(br[c])));
        }
    } else {
        float q = 0.0f;
        for (int64_t c = threadIdx.x; c < a.cols; c += blockDim.x) {
            const float v = to_f32(xr[c]);
            q = __fadd_rn(q, __fmul_rn(v, v));
        }
        const float ms = __fdiv_rn(cta_reduce<false>(q, red), n);
        const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, a.eps)));
        for (int64_t c = threadIdx.x; c < a.cols; c += blockDim.x)
            yr[c] = from_f32<T>(__fmul_rn(__fmul_rn(to_f32(xr[c]), rstd), to_f32(wr[c])));
    }
}

// variant v: u = v % 12 gives threads-per-row = base << (u / 3) for u / 3 in 0..3 and CTA threads =
// {128, 256, 512}[u % 3], where base = fewest threads whose registers hold the row (min 32);
// v / 12 = 0: rows loaded straight into registers, 1: persistent CTAs fed by a bulk-copy ring.
constexpr int ROW_VARIANTS = 24;
constexpr int kAutoVariant = 3;  // threads-per-row = base * 2, 128-thread CTAs, direct loads

template <typename T, int V, int OP>
int launch_pipe(const RowArgs &a, int cta, cudaStream_t st, const char *name) {
    PipeArgs p{a, 2, device_error_word()};
    if (!p.error) return fail(ENC_ERR_NO_MEMORY, "%s: cannot allocate the device status word", name);
    const int R = cta / a.tpr;
    const size_t stage_bytes = (size_t)R * a.cols * sizeof(T);
    const size_t budget = cta <= 128 ? 48 * 1024 : (cta <= 256 ? 64 * 1024 : 96 * 1024);
    int stages = (int)(budget / stage_bytes);
    if (stages < 2) stages = 2;
    if (stages > 16) stages = 16;
    p.stages = stages;
    const size_t smem = stage_bytes * stages;
    auto kern = row_pipe_kernel<T, V, OP>;
    static std::mutex mu;
    static std::map<std::tuple<const void *, int, size_t, int>, int> occupancy;  // per device too
    int dev = 0;
    cudaGetDevice(&dev);
    int per_sm = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        auto key = std::make_tuple((const void *)kern, cta, smem, dev);
        auto it = occupancy.find(key);
        if (it == occupancy.end()) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, cta, smem);
            if (e != cudaSuccess || per_sm < 1) {
                cudaGetLastError();
                return fail(ENC_ERR_UNSUPPORTED, "%s: the bulk-copy variant does not fit (%zu bytes of shared memory per CTA)", name, smem);
            }
            occupancy[key] = per_sm;
        } else {
            per_sm = it->second;
        }
    }
    const int64_t nblocks = cdiv(a.rows, R);
    int64_t grid = (int64_t)device_props().sm_count * per_sm;
    if (grid > nblocks) grid = nblocks;
    kern<<<(unsigned)grid, cta, smem, st>>>(p);
    return check_launch(name);
}

template <typename T, int OP>
int launch_pipe_v(const RowArgs &a, int v, int cta, cudaStream_t st, const char *name) {
    switch (v) {
        case 1: return launch_pipe<T, 1, OP>(a, cta, st, name);
        case 2: return launch_pipe<T, 2, OP>(a, cta, st, name);
        case 4: return launch_pipe<T, 4, OP>(a, cta, st, name);
        case 8: return launch_pipe<T, 8, OP>(a, cta, st, name);
        default: return fail(ENC_ERR_UNSUPPORTED, "%s: the bulk-copy variant holds at most 8 vectors per thread", name);
    }
}

template <typename T, int OP, bool VEC>
int launch_v(const RowArgs &a, int v, int cta, cudaStream_t st) {
    const unsigned grid = (unsigned)cdiv(a.rows, cta / a.tpr);
    switch (v) {
        case 1: launch_overlapped(row_kernel<T, 1, VEC, OP>, grid, cta, 0, st, a); break;
        case 2: launch_overlapped(row_kernel<T, 2, VEC, OP>, grid, cta, 0, st, a); break;
        case 4: launch_overlapped(row_kernel<T, 4, VEC, OP>, grid, cta, 0, st, a); break;
        case 8: launch_overlapped(row_kernel<T, 8, VEC, OP>, grid, cta, 0, st, a); break;
        case 16:
            if constexpr (sizeof(T) == 2) {
                launch_overlapped(row_kernel<T, 16, VEC, OP>, grid, cta, 0, st, a);
                break;
            }
            [[fallthrough]];
        default: return fail(ENC_ERR_UNSUPPORTED, "row kernel: no instantiation for %d vectors per thread", v);
    }
    return ENC_OK;
}

template <typename T, int OP>
int launch_rows(RowArgs a, int variant, cudaStream_t st, const char *name) {
    constexpr int NV = Pack<T>::N;
    // At most 8 raw vectors (32 registers) of float32 row data per thread, 16 (64 registers) of packed
    // float16/bfloat16: the widest row one warp holds is 1024 float32 or 4096 half values.
    constexpr int MAXV = sizeof(T) == 4 ? 8 : 16;
    if (a.rows == 0 || a.cols == 0) return ENC_OK;
    if (a.rows > 0x7fffffffLL) return fail(ENC_ERR_UNSUPPORTED, "%s: more than 2^31-1 rows", name);
    if (variant >= ROW_VARIANTS) return fail(ENC_ERR_BAD_ARG, "%s: variant %d out of range", name, variant);
    // measured (TB/s): RMSNorm bf16 [16384, 4096] is fastest with four times the minimum threads per row (6.5 against
    // 6.1), LayerNorm bf16 with twice (5.93 against 4.86 and 4.52), softmax fp32 [4096, 1024] and [4096, 4096] with the
    // minimum (5.29, 6.33).  float32 rows of 4096 (16 KB): LayerNorm and RMSNorm with the minimum, 8 vectors per thread
    // (5.98 and 6.20 against 5.24 and 5.83 with twice).  Wide 16-bit softmax rows take twice the minimum, 64 elements
    // per thread with the exponentials kept in registers (5.07 against 4.57 with four times and 4.46 with the minimum).
    if (variant < 0) {
        if (OP == OP_SOFTMAX) variant = sizeof(T) == 2 && a.cols > 2048 ? 3 : 0;
        else if (OP == OP_LAYERNORM) variant = sizeof(T) == 4 && a.cols >= 2048 ? 0 : kAutoVariant;
        else variant = sizeof(T) == 4 ? (a.cols >= 2048 ? 0 : 3) : (a.cols * (int64_t)sizeof(T) >= 4096 ? 6 : kAutoVariant);
    }
    const bool pipe = variant >= 12;
    const int shift = (variant % 12) / 3;
    int cta = 128 << (variant % 3);
    int64_t tpr64 = next_pow2(cdiv(a.cols, (int64_t)NV * MAXV));
    if (tpr64 < 32) tpr64 = 32;
    tpr64 <<= shift;
    if (tpr64 > 512) {
        if (tpr64 >> shift > 512) {  // does not fit in registers even at 512 threads per row
            row_kernel_wide<T, OP><<<(unsigned)a.rows, 1024, 0, st>>>(a);
            return check_launch(name);
        }
        tpr64 = 512;
    }
    a.tpr = (int)tpr64;
    if (cta < a.tpr) cta = a.tpr;
    // The reductions of a row that spans two warps are CTA barriers, which hold up the other rows of the CTA as well,
    // and LayerNorm's CTA-wide agreement on the ill-conditioned branch costs a second barrier per row unless the CTA
    // holds one row: at the smallest CTA size such a row gets a CTA of its own (LayerNorm bf16 [16384, 4096]: 6.01
    // against 5.93 TB/s; softmax fp16 [4096, 4096]: 5.30 against 5.11).
    if (!pipe && a.tpr == 64 && variant % 3 == 0) cta = 64;
    int v = next_pow2(cdiv(a.cols, (int64_t)a.tpr * NV));
    const bool vec = a.cols % NV == 0 && a.stride_x % NV == 0 && a.stride_y % NV == 0 &&
                     aligned16(a.x) && aligned16(a.y) &&
                     (OP == OP_SOFTMAX || aligned16(a.w)) && (OP != OP_LAYERNORM || aligned16(a.b));
    if (pipe && vec && v <= 8) return launch_pipe_v<T, OP>(a, v, cta, st, name);
    int rc = vec ? launch_v<T, OP, true>(a, v, cta, st) : launch_v<T, OP, false>(a, v, cta, st);
    if (rc != ENC_OK) return rc;
    return check_launch(name);
}

template <int OP> int dispatch(const RowArgs &a, int dtype, int variant, void *stream, const char *name) {
    if (!a.x || !a.y) return fail(ENC_ERR_BAD_ARG, "%s: NULL input or output", name);
    if (a.rows < 0 || a.cols < 0) return fail(ENC_ERR_BAD_ARG, "%s: negative shape", name);
    if (a.stride_x < a.cols && a.rows > 1) return fail(ENC_ERR_BAD_ARG, "%s: row stride %lld is smaller than the row length %lld", name, (long long)a.stride_x, (long long)a.cols);
    switch (dtype) {
        case ENC_F32: return launch_rows<float, OP>(a, variant, as_stream(stream), name);
        case ENC_F16: return launch_rows<__half, OP>(a, variant, as_stream(stream), name);
        case ENC_BF16: return launch_rows<__nv_bfloat16, OP>(a, variant, as_stream(stream), name);
        default: return fail(ENC_ERR_BAD_ARG, "%s: dtype %d is not float32, float16 or bfloat16", name, dtype);
    }
}

}  // namespace

int row_variants() { return ROW_VARIANTS; }
void row_variant_info(int v, char *out, size_t n) {
    snprintf(out, n, "threads_per_row=base*%d cta_threads=%d %s (base = fewest threads whose registers hold the row, min 32; a row of 64 threads takes a 64-thread CTA at cta_threads=128)",
             1 << ((v % 12) / 3), 128 << (v % 3), v >= 12 ? "persistent CTAs fed by a cp.async.bulk ring" : "direct loads");
}

}  // namespace enc

extern "C" int enc_softmax(const void *in, void *out, int64_t rows, int64_t cols, int64_t stride_in,
                           int64_t stride_out, int dtype, int variant, void *stream) {
    ENC_PROLOGUE();
    enc::RowArgs a{in, out, nullptr, nullptr, nullptr, nullptr, rows, cols, stride_in, stride_out, 0.f, 32};
    return enc::dispatch<enc::OP_SOFTMAX>(a, dtype, variant, stream, "enc_softmax");
}

extern "C" int enc_layernorm(const void *x, void *y, const void *w, const void *b, float *mean,
                             float *rstd, int64_t rows, int64_t cols, int64_t stride_x,
                             int64_t stride_y, float eps, int dtype, int variant, void *stream) {
    ENC_PROLOGUE();
    if (!w || !b) return enc::fail(ENC_ERR_BAD_ARG, "enc_layernorm: NULL weight or bias");
    enc::RowArgs a{x, y, w, b, mean, rstd, rows, cols, stride_x, stride_y, eps, 32};
    return enc::dispatch<enc::OP_LAYERNORM>(a, dtype, variant, stream, "enc_layernorm");
}

extern "C" int enc_rmsnorm(const void *x, const void *w, void *y, int64_t rows, int64_t cols,
                           int64_t stride_x, int64_t stride_y, float eps, int dtype, int variant,
                           void *stream) {
    ENC_PROLOGUE();
    if (!w) return enc::fail(ENC_ERR_BAD_ARG, "enc_rmsnorm: NULL weight");
    enc::RowArgs a{x, y, w, nullptr, nullptr, nullptr, rows, cols, stride_x, stride_y, eps, 32};
    return enc::dispatch<enc::OP_RMSNORM>(a, dtype, variant, stream, "enc_rmsnorm");
}
