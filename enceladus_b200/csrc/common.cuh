// Shared host/device helpers of the sm_100a kernel library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/enceladus_b200.h"

namespace enc {

// ---- host-side status plumbing -------------------------------------------------------------
int fail(int status, const char *fmt, ...);  // sets the thread-local message, returns status
bool take_forced_failure(int *status);        // enc_test_fail_next hook
int check_launch(const char *what);           // cudaGetLastError -> status

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

struct DeviceProps {
    int device = -1;
    int sm_count = 148;
    int max_smem_optin = 0;
    int l2_bytes = 0;
};
const DeviceProps &device_props();  // cached per current device

// Word 0 of the per-device status block is set by a kernel whose bounded wait ran out.
unsigned int *device_error_word();  // device pointer (allocated on first use), or nullptr

inline size_t dtype_size(int dt) {
    switch (dt) {
        case ENC_F32: case ENC_I32: return 4;
        case ENC_F16: case ENC_BF16: case ENC_I16: return 2;
        case ENC_I8: case ENC_U8: return 1;
        case ENC_I64: return 8;
        default: return 0;
    }
}
inline bool is_float_dtype(int dt) { return dt == ENC_F32 || dt == ENC_F16 || dt == ENC_BF16; }
__host__ __device__ inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int next_pow2(int64_t n) {
    int p = 1;
    while (p < n) p <<= 1;
    return p;
}

#define ENC_PROLOGUE()                              \
    do {                                            \
        int forced_;                                \
        if (enc::take_forced_failure(&forced_)) return forced_; \
    } while (0)

// ---- device helpers ------------------------------------------------------------------------
#ifdef __CUDACC__

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(int v) { return __int2float_rn(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// 16-byte vector of T unpacked to float registers and back.
template <typename T> struct Pack;
template <> struct Pack<float> {
    static constexpr int N = 4;
    __device__ __forceinline__ static void unpack(const uint4 &u, float *f) {
        f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
    }
    __device__ __forceinline__ static uint4 pack(const float *f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                          __float_as_uint(f[3]));
    }
};
template <> struct Pack<__half> {
    static constexpr int N = 8;
    __device__ __forceinline__ static void unpack(const uint4 &u, float *f) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __half22float2(h[i]);
            f[2 * i] = t.x; f[2 * i + 1] = t.y;
        }
    }
    __device__ __forceinline__ static uint4 pack(const float *f) {
        uint4 u;
        __half2 *h = reinterpret_cast<__half2 *>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        return u;
    }
};
template <> struct Pack<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ __forceinline__ static void unpack(const uint4 &u, float *f) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // bf16 -> f32 is a 16-bit shift
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static uint4 pack(const float *f) {
        uint4 u;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        return u;
    }
};

// Packed float32 pairs: sm_100 executes fma / add on two float32 values in one instruction.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// ---- programmatic dependent launch ----------------------------------------------------------------
// A kernel launched with launch_overlapped() may start while the kernel before it on the stream is still
// running; it must execute grid_dependency_wait() before its first access to global memory, which
// returns once that kernel has completed and its writes are visible.  What overlaps is the launch
// latency and the index arithmetic in front of the wait - about a microsecond, which matters for kernels
// that run for less than ten.  Stream order as the caller sees it is unchanged.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.launch_dependents;\n\tgriddepcontrol.wait;" ::: "memory");
}
template <typename... KArgs, typename... Args>
inline void launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Streaming 128-bit accesses: read-once / write-once data should not displace L2-resident
// operands (weights, bias) nor wait on L1 allocation.
__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(void *p, const uint4 &v) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// 2^x by the special-function unit (relative error about 2^-22; results below 2^-126 flush to zero).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

#endif  // __CUDACC__

}  // namespace enc
