// Histogram for sm_100a: shared-memory-privatised atomics, one flush per CTA.
//
// The reference issues one global atomic per element (examples/09_histogram.py:17-24,
// src/enceladus/compiler/codegen/atomic.py:1-25) and is contention-bound.  Here each persistent CTA
// keeps R replicas of the histogram in shared memory, laid out as hist[bin * R + (lane % R)], so
// lanes of a warp that hit the same bin land on different addresses (and, for R = 32, different
// banks); counts are flushed to the int32 output with one global atomicAdd per non-zero bin per
// CTA.  The input is read once with 128-bit streaming loads: the kernel is HBM-bound when the
// shared-memory atomics keep up, which is what R is for.
//
// The bin index is computed exactly as the reference does, in float32:
//   b = floor((float(x) - lo) * inv_width) -> int32 (saturating, NaN -> 0); counted iff 0 <= b < bins.
// Integer addition commutes, so the counts are bit-exact whatever the order.  The kernel is
// instruction-issue bound before it is atomics bound, so the per-element path is kept to a handful of
// instructions (one unsigned range compare, one address computation, one shared atomic).
#include <type_traits>

#include "common.cuh"

namespace enc {
namespace {

struct HistArgs {
    const void *x;
    int *hist;
    int64_t n;
    float lo, inv_width;
    int num_bins;
    int rshift;  // log2(R)
};

__device__ __forceinline__ int bin_of(float xf, float lo, float inv_width) {
    // cvt.rmi.s32.f32 rounds toward -inf (= floor), saturates, and maps NaN to 0, which is the
    // reference's floor followed by its saturating float->int32 conversion.
    return __float2int_rd(__fmul_rn(__fsub_rn(xf, lo), inv_width));
}

template <typename T> struct Elems;  // 16-byte vector -> float values
template <> struct Elems<float> { static constexpr int N = 4; __device__ static void get(const uint4 &u, float *f) { Pack<float>::unpack(u, f); } };
template <> struct Elems<__half> { static constexpr int N = 8; __device__ static void get(const uint4 &u, float *f) { Pack<__half>::unpack(u, f); } };
template <> struct Elems<__nv_bfloat16> { static constexpr int N = 8; __device__ static void get(const uint4 &u, float *f) { Pack<__nv_bfloat16>::unpack(u, f); } };
template <> struct Elems<int> {
    static constexpr int N = 4;
    __device__ static void get(const uint4 &u, float *f) {
        f[0] = __int2float_rn((int)u.x); f[1] = __int2float_rn((int)u.y);
        f[2] = __int2float_rn((int)u.z); f[3] = __int2float_rn((int)u.w);
    }
};

// IDENTITY: int32 input with lo == 0 and inv_width == 1, where floor((float(x) - 0) * 1) == x for every
// x that can land in a bin (bins <= 2^24, so the int -> float conversion is exact there and monotone
// elsewhere); the bin is the value itself and the float pipeline is skipped.  Same counts, fewer
// instructions: at HBM speed an int32 element has a budget of about twenty lane-instructions.
template <typename T, int UNROLL, bool IDENTITY>
__global__ void __launch_bounds__(1024) hist_kernel(HistArgs a) {
    extern __shared__ int sh[];
    constexpr int NV = Elems<T>::N;
    const int R = 1 << a.rshift;
    const int total = a.num_bins << a.rshift;
    for (int i = threadIdx.x; i < total; i += blockDim.x) sh[i] = 0;
    __syncthreads();

    const int rshift = a.rshift;
    const int rep = threadIdx.x & (R - 1);
    const unsigned nbins = (unsigned)a.num_bins;
    const float lo = a.lo, inv_width = a.inv_width;
    const T *x = reinterpret_cast<const T *>(a.x);
    // The base pointer may be unaligned: peel scalar elements up to the first 16-byte boundary.
    int64_t head = (int64_t)(((16 - (reinterpret_cast<uintptr_t>(x) & 15)) & 15) / sizeof(T));
    if (head > a.n) head = a.n;
    const int64_t nvec = (a.n - head) / NV;
    const uint4 *xv = reinterpret_cast<const uint4 *>(x + head);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;

    auto count_bin = [&](int b) {
        if ((unsigned)b < nbins) atomicAdd(&sh[(b << rshift) + rep], 1);  // one unsigned compare covers b < 0
    };
    auto count_vec = [&](const uint4 &raw) {
        if (IDENTITY) {
            count_bin((int)raw.x); count_bin((int)raw.y); count_bin((int)raw.z); count_bin((int)raw.w);
        } else {
            float f[NV];
            Elems<T>::get(raw, f);
#pragma unroll
            for (int e = 0; e < NV; ++e) count_bin(bin_of(f[e], lo, inv_width));
        }
    };

    for (int64_t v0 = tid; v0 < nvec; v0 += stride * UNROLL) {
        uint4 raw[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
            if (v0 + u * stride < nvec) raw[u] = ld_stream(xv + v0 + u * stride);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
            if (v0 + u * stride < nvec) count_vec(raw[u]);
    }
    // scalar head and tail (each shorter than one vector)
    if (blockIdx.x == 0 && threadIdx.x < 32) {
        const int64_t tail0 = head + nvec * NV;
        const int lane = threadIdx.x;
        if (lane < head) count_bin(bin_of(to_f32(x[lane]), lo, inv_width));
        if (tail0 + lane < a.n) count_bin(bin_of(to_f32(x[tail0 + lane]), lo, inv_width));
    }

    __syncthreads();
    for (int b = threadIdx.x; b < a.num_bins; b += blockDim.x) {
        int c = 0;
        for (int r = 0; r < R; ++r) c += sh[(b << a.rshift) + ((r + threadIdx.x) & (R - 1))];
        if (c) atomicAdd(&a.hist[b], c);
    }
}

// More bins than shared memory can hold: one global atomic per element, like the reference.
template <typename T>
__global__ void __launch_bounds__(256) hist_global_kernel(const T *x, int *hist, int64_t n, float lo,
                                                          float inv_width, int64_t num_bins) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int b = bin_of(to_f32(x[i]), lo, inv_width);
        if (b >= 0 && b < num_bins) atomicAdd(&hist[b], 1);
    }
}

// variant v: cta_threads = {1024, 512}[v & 1], vectors in flight per thread = {4, 2}[(v >> 1) & 1],
// resident CTAs per SM = {2048/threads, half of that}[(v >> 2) & 1] (fewer CTAs = more replicas each)
constexpr int HIST_VARIANTS = 8;
constexpr int kMaxSmem = 200 * 1024;

template <typename T>
int launch_hist(HistArgs a, int variant, cudaStream_t st) {
    const DeviceProps &dp = device_props();
    if ((int64_t)a.num_bins * 4 > kMaxSmem) {
        int64_t g = cdiv(a.n, 256);
        if (g > (int64_t)dp.sm_count * 32) g = (int64_t)dp.sm_count * 32;
        hist_global_kernel<T><<<(unsigned)g, 256, 0, st>>>((const T *)a.x, a.hist, a.n, a.lo, a.inv_width, a.num_bins);
        return check_launch("enc_histogram");
    }
    const int v = variant < 0 ? 0 : variant;
    const int threads = (v & 1) ? 512 : 1024;
    const bool unroll2 = (v >> 1) & 1;
    int ctas_per_sm = (2048 / threads) >> ((v >> 2) & 1);
    const int budget = kMaxSmem / ctas_per_sm;
    int rshift = 5;
    while (rshift > 0 && ((int64_t)a.num_bins << rshift) * 4 > budget) --rshift;
    a.rshift = rshift;
    const size_t smem = ((size_t)a.num_bins << rshift) * 4;
    int64_t g = (int64_t)dp.sm_count * ctas_per_sm;
    const int64_t need = cdiv(a.n, (int64_t)threads * Elems<T>::N);
    if (g > need) g = need > 0 ? need : 1;
    // the bin is the value itself: int32 input, unit-width bins starting at zero
    const bool identity = std::is_same<T, int>::value && a.lo == 0.0f && a.inv_width == 1.0f && a.num_bins <= (1 << 24);
    void (*kern)(HistArgs) = nullptr;
    if constexpr (std::is_same<T, int>::value) {
        if (identity) kern = unroll2 ? hist_kernel<T, 2, true> : hist_kernel<T, 4, true>;
    }
    if (!kern) kern = unroll2 ? hist_kernel<T, 2, false> : hist_kernel<T, 4, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return fail(ENC_ERR_LAUNCH, "enc_histogram: cannot opt in to %d bytes of shared memory: %s", kMaxSmem, cudaGetErrorString(e));
    kern<<<(unsigned)g, threads, smem, st>>>(a);
    return check_launch("enc_histogram");
}

}  // namespace

int hist_variants() { return HIST_VARIANTS; }
void hist_variant_info(int v, char *out, size_t n) {
    const int threads = (v & 1) ? 512 : 1024;
    snprintf(out, n, "cta_threads=%d vectors_in_flight=%d ctas_per_sm=%d (replicas = largest power of two that fits, max 32)",
             threads, (v >> 1) & 1 ? 2 : 4, (2048 / threads) >> ((v >> 2) & 1));
}

}  // namespace enc

extern "C" int enc_histogram(const void *x, int32_t *hist, int64_t n, float lo, float inv_width,
                             int64_t num_bins, int dtype, int variant, void *stream) {
    ENC_PROLOGUE();
    if (!hist || (!x && n > 0)) return enc::fail(ENC_ERR_BAD_ARG, "enc_histogram: NULL pointer");
    if (n < 0 || num_bins <= 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_histogram: n must be >= 0 and num_bins > 0");
    if (num_bins > 0x7fffffffLL) return enc::fail(ENC_ERR_UNSUPPORTED, "enc_histogram: more than 2^31-1 bins");
    if (variant >= enc::HIST_VARIANTS) return enc::fail(ENC_ERR_BAD_ARG, "enc_histogram: variant %d out of range", variant);
    if (n == 0) return ENC_OK;
    enc::HistArgs a{x, hist, n, lo, inv_width, (int)num_bins, 0};
    cudaStream_t st = enc::as_stream(stream);
    switch (dtype) {
        case ENC_F32: return enc::launch_hist<float>(a, variant, st);
        case ENC_F16: return enc::launch_hist<__half>(a, variant, st);
        case ENC_BF16: return enc::launch_hist<__nv_bfloat16>(a, variant, st);
        case ENC_I32: return enc::launch_hist<int>(a, variant, st);
        default: return enc::fail(ENC_ERR_BAD_ARG, "enc_histogram: dtype %d is not float32, float16, bfloat16 or int32", dtype);
    }
}
