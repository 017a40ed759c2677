// Fused GELU (erf and tanh forms, optional scale and per-column bias) and vector add for sm_100a.
//
// HBM-bound: one read and one write per element.  Each thread keeps UNROLL independent 128-bit
// streaming loads in flight; the grid is sized to a whole number of waves over the SMs and strides
// over the array.  The expression is evaluated exactly as the reference kernel writes it
// (examples/05_fused_gelu.py:22-25): t = x*scale + bias (two roundings), then
// 0.5*t*(1+erf(t*0.70710677f)), every product and sum rounded to float32 on its own.
#include "common.cuh"

namespace enc {
namespace {

enum { GELU_ERF = 0, GELU_TANH = 1 };

template <int MODE> __device__ __forceinline__ float gelu(float t) {
    if (MODE == GELU_ERF) {
        const float e = erff(__fmul_rn(t, 0.70710677f));
        return __fmul_rn(__fmul_rn(0.5f, t), __fadd_rn(1.0f, e));
    } else {
        // 0.7978845608 * (t + 0.044715*t*t*t), left to right
        const float c = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, t), t), t);
        const float inner = __fmul_rn(0.7978845608f, __fadd_rn(t, c));
        return __fmul_rn(__fmul_rn(0.5f, t), __fadd_rn(1.0f, tanhf(inner)));
    }
}

struct GeluArgs {
    const void *x;
    const void *bias;
    void *out;
    int64_t n, n_cols;
    float scale;
    int has_scale;
};

template <typename T, int MODE, bool BIAS, int UNROLL>
__global__ void __launch_bounds__(256) gelu_vec_kernel(GeluArgs a) {
    constexpr int NV = Pack<T>::N;
    const T *x = reinterpret_cast<const T *>(a.x);
    const T *bias = reinterpret_cast<const T *>(a.bias);
    T *out = reinterpret_cast<T *>(a.out);
    const int64_t nvec = a.n / NV;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * UNROLL) {
        uint4 raw[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t v = v0 + u * stride;
            if (v < nvec) raw[u] = ld_stream(x + v * NV);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t v = v0 + u * stride;
            if (v >= nvec) continue;
            float f[NV];
            Pack<T>::unpack(raw[u], f);
            int64_t col = BIAS ? (v * NV) % a.n_cols : 0;
#pragma unroll
            for (int e = 0; e < NV; ++e) {
                float t = f[e];
                if (a.has_scale) t = __fmul_rn(t, a.scale);
                if (BIAS) {
                    t = __fadd_rn(t, to_f32(__ldg(bias + col)));
                    if (++col == a.n_cols) col = 0;
                }
                f[e] = gelu<MODE>(t);
            }
            st_stream(out + v * NV, Pack<T>::pack(f));
        }
    }
    // ragged tail (fewer than NV elements)
    const int64_t tail = nvec * NV + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tail < a.n) {
        float t = to_f32(x[tail]);
        if (a.has_scale) t = __fmul_rn(t, a.scale);
        if (BIAS) t = __fadd_rn(t, to_f32(bias[tail % a.n_cols]));
        out[tail] = from_f32<T>(gelu<MODE>(t));
    }
}

// Unaligned base pointers: plain scalar grid-stride loop.
template <typename T, int MODE, bool BIAS>
__global__ void __launch_bounds__(256) gelu_scalar_kernel(GeluArgs a) {
    const T *x = reinterpret_cast<const T *>(a.x);
    const T *bias = reinterpret_cast<const T *>(a.bias);
    T *out = reinterpret_cast<T *>(a.out);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
        float t = to_f32(x[i]);
        if (a.has_scale) t = __fmul_rn(t, a.scale);
        if (BIAS) t = __fadd_rn(t, to_f32(bias[i % a.n_cols]));
        out[i] = from_f32<T>(gelu<MODE>(t));
    }
}

// variant v: unroll = {4, 2, 1, 8}[v % 4] vectors in flight per thread, waves = {8, 16, 4}[v / 4] CTAs per SM
constexpr int GELU_VARIANTS = 12;
constexpr int kUnroll[4] = {4, 2, 1, 8};
constexpr int kWaves[3] = {8, 16, 4};

template <typename T, int MODE, bool BIAS>
int launch_gelu(const GeluArgs &a, int variant, cudaStream_t st) {
    constexpr int NV = Pack<T>::N;
    const int sms = device_props().sm_count;
    const int v = variant < 0 ? 0 : variant;
    const int unroll = kUnroll[v % 4];
    const int64_t max_grid = (int64_t)sms * kWaves[v / 4];
    if (!aligned16(a.x) || !aligned16(a.out)) {
        const int64_t g = cdiv(a.n, 256);
        gelu_scalar_kernel<T, MODE, BIAS><<<(unsigned)(g < max_grid ? g : max_grid), 256, 0, st>>>(a);
        return check_launch("enc_gelu");
    }
    const int64_t nvec = a.n / NV;
    int64_t g = cdiv(nvec > 0 ? nvec : 1, (int64_t)256 * unroll);
    if (g > max_grid) g = max_grid;
    if (g < 1) g = 1;
    switch (unroll) {
        case 1: gelu_vec_kernel<T, MODE, BIAS, 1><<<(unsigned)g, 256, 0, st>>>(a); break;
        case 2: gelu_vec_kernel<T, MODE, BIAS, 2><<<(unsigned)g, 256, 0, st>>>(a); break;
        case 4: gelu_vec_kernel<T, MODE, BIAS, 4><<<(unsigned)g, 256, 0, st>>>(a); break;
        default: gelu_vec_kernel<T, MODE, BIAS, 8><<<(unsigned)g, 256, 0, st>>>(a); break;
    }
    return check_launch("enc_gelu");
}

template <typename T> int gelu_mode(const GeluArgs &a, int mode, int variant, cudaStream_t st) {
    const bool bias = a.bias != nullptr;
    if (mode == GELU_ERF) return bias ? launch_gelu<T, GELU_ERF, true>(a, variant, st) : launch_gelu<T, GELU_ERF, false>(a, variant, st);
    return bias ? launch_gelu<T, GELU_TANH, true>(a, variant, st) : launch_gelu<T, GELU_TANH, false>(a, variant, st);
}

// ---- vector add ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) add_kernel(const T *x, const T *y, T *out, int64_t n, bool vec) {
    constexpr int NV = Pack<T>::N;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        const int64_t nvec = n / NV;
        for (int64_t v = tid; v < nvec; v += stride) {
            float a[NV], b[NV];
            Pack<T>::unpack(ld_stream(x + v * NV), a);
            Pack<T>::unpack(ld_stream(y + v * NV), b);
#pragma unroll
            for (int e = 0; e < NV; ++e) a[e] = __fadd_rn(a[e], b[e]);
            st_stream(out + v * NV, Pack<T>::pack(a));
        }
        const int64_t tail = nvec * NV + tid;
        if (tail < n) out[tail] = from_f32<T>(__fadd_rn(to_f32(x[tail]), to_f32(y[tail])));
    } else {
        for (int64_t i = tid; i < n; i += stride) out[i] = from_f32<T>(__fadd_rn(to_f32(x[i]), to_f32(y[i])));
    }
}

template <typename T> int launch_add(const void *x, const void *y, void *out, int64_t n, cudaStream_t st) {
    const bool vec = aligned16(x) && aligned16(y) && aligned16(out);
    int64_t g = cdiv(n, 256 * (vec ? Pack<T>::N : 1));
    const int64_t max_grid = (int64_t)device_props().sm_count * 16;
    if (g > max_grid) g = max_grid;
    add_kernel<T><<<(unsigned)g, 256, 0, st>>>((const T *)x, (const T *)y, (T *)out, n, vec);
    return check_launch("enc_add");
}

}  // namespace

int gelu_variants() { return GELU_VARIANTS; }
void gelu_variant_info(int v, char *out, size_t n) {
    snprintf(out, n, "vectors_in_flight=%d ctas_per_sm=%d cta_threads=256", kUnroll[v % 4], kWaves[v / 4]);
}

}  // namespace enc

extern "C" int enc_gelu(const void *x, const void *bias, void *out, int64_t n, int64_t n_cols,
                        float scale, int has_scale, int mode, int dtype, int variant, void *stream) {
    ENC_PROLOGUE();
    if (!x || !out) return enc::fail(ENC_ERR_BAD_ARG, "enc_gelu: NULL input or output");
    if (n < 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_gelu: negative length");
    if (mode != 0 && mode != 1) return enc::fail(ENC_ERR_BAD_ARG, "enc_gelu: mode must be 0 (erf) or 1 (tanh), got %d", mode);
    if (bias && n_cols <= 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_gelu: a bias needs n_cols > 0");
    if (variant >= enc::GELU_VARIANTS) return enc::fail(ENC_ERR_BAD_ARG, "enc_gelu: variant %d out of range", variant);
    if (n == 0) return ENC_OK;
    enc::GeluArgs a{x, bias, out, n, n_cols, scale, has_scale};
    cudaStream_t st = enc::as_stream(stream);
    switch (dtype) {
        case ENC_F32: return enc::gelu_mode<float>(a, mode, variant, st);
        case ENC_F16: return enc::gelu_mode<__half>(a, mode, variant, st);
        case ENC_BF16: return enc::gelu_mode<__nv_bfloat16>(a, mode, variant, st);
        default: return enc::fail(ENC_ERR_BAD_ARG, "enc_gelu: dtype %d is not float32, float16 or bfloat16", dtype);
    }
}

extern "C" int enc_add(const void *x, const void *y, void *out, int64_t n, int dtype, int variant,
                       void *stream) {
    ENC_PROLOGUE();
    (void)variant;
    if (!x || !y || !out) return enc::fail(ENC_ERR_BAD_ARG, "enc_add: NULL pointer");
    if (n < 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_add: negative length");
    if (n == 0) return ENC_OK;
    cudaStream_t st = enc::as_stream(stream);
    switch (dtype) {
        case ENC_F32: return enc::launch_add<float>(x, y, out, n, st);
        case ENC_F16: return enc::launch_add<__half>(x, y, out, n, st);
        case ENC_BF16: return enc::launch_add<__nv_bfloat16>(x, y, out, n, st);
        default: return enc::fail(ENC_ERR_BAD_ARG, "enc_add: dtype %d is not float32, float16 or bfloat16", dtype);
    }
}
