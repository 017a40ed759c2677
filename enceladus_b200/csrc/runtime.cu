// Host-side runtime of the kernel library: status strings, device properties, the device error
// word that bounded device-side waits raise, variant tables and synchronisation.
#include <mutex>

#include "sm100.cuh"

namespace enc {

int row_variants();
void row_variant_info(int v, char *out, size_t n);
int gelu_variants();
void gelu_variant_info(int v, char *out, size_t n);
int hist_variants();
void hist_variant_info(int v, char *out, size_t n);
int scan_variants();
void scan_variant_info(int v, char *out, size_t n);
int matmul_variants();
void matmul_variant_info(int v, char *out, size_t n);
int attention_variants();
void attention_variant_info(int v, char *out, size_t n);
int int_matmul_variants();
void int_matmul_variant_info(int v, char *out, size_t n);

namespace {
thread_local char g_error[1024] = "";
thread_local int g_forced = 0;
constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
DeviceProps g_props[MAX_DEVICES];
unsigned int *g_error_word[MAX_DEVICES];
}  // namespace

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}

bool take_forced_failure(int *status) {
    if (!g_forced) return false;
    *status = g_forced;
    g_forced = 0;
    fail(*status, "failure injected by enc_test_fail_next(%d)", *status);
    return true;
}

int check_launch(const char *what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return ENC_OK;
    return fail(ENC_ERR_LAUNCH, "%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
}

const DeviceProps &device_props() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= MAX_DEVICES) dev = 0;
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceProps &p = g_props[dev];
    if (p.device != dev) {
        p.device = dev;
        cudaDeviceGetAttribute(&p.sm_count, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&p.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        cudaDeviceGetAttribute(&p.l2_bytes, cudaDevAttrL2CacheSize, dev);
        if (p.sm_count <= 0) p.sm_count = 148;
    }
    return p;
}

unsigned int *device_error_word() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= MAX_DEVICES) return nullptr;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_error_word[dev]) {
        unsigned int *p = nullptr;  // first use on this device; must not happen inside a stream capture
        if (cudaMalloc(&p, 256) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cudaMemset(p, 0, 256);
        g_error_word[dev] = p;
    }
    return g_error_word[dev];
}

bool make_tensor_map(CUtensorMap *map, const void *base, int elem, int rank, const uint64_t *dims,
                     const uint64_t *strides_bytes, const uint32_t *box, char *err, size_t errlen) {
    using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
            cudaGetLastError();
            snprintf(err, errlen, "the driver does not provide cuTensorMapEncodeTiled");
            return false;
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        e[i] = 1;
        if (i + 1 < rank) s[i] = strides_bytes[i];
    }
    const CUtensorMapDataType dt = elem == TMAP_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : elem == TMAP_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = encode(map, dt,
                              (cuuint32_t)rank, const_cast<void *>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(err, errlen, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu, box %u x %u)",
                 (int)r, rank, (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
        return false;
    }
    return true;
}

}  // namespace enc

namespace enc {
namespace {
// Polls a word that nothing ever sets, `polls` times at most, then gives up the way every bounded
// device-side wait of the library does: it raises the device status word and returns.
__global__ void wait_timeout_kernel(const unsigned int *never_set, unsigned int *error, unsigned int polls) {
    unsigned int seen = 0;
    for (unsigned int i = 0; i < polls && !seen; ++i) {
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(never_set) : "memory");
        __nanosleep(1000);
    }
    if (!seen) atomicExch(error, 6u);
}
}  // namespace
}  // namespace enc

extern "C" int enc_test_device_wait(unsigned int polls, void *stream) {
    ENC_PROLOGUE();
    if (polls > 1000000u) return enc::fail(ENC_ERR_BAD_ARG, "enc_test_device_wait: at most 1000000 polls (about one second)");
    unsigned int *block = enc::device_error_word();
    if (!block) return enc::fail(ENC_ERR_NO_MEMORY, "enc_test_device_wait: cannot allocate the device status word");
    enc::wait_timeout_kernel<<<1, 1, 0, enc::as_stream(stream)>>>(block + 8, block, polls);  // word 8 of the block stays zero
    return enc::check_launch("enc_test_device_wait");
}

extern "C" const char *enc_last_error(void) { return enc::g_error; }

extern "C" void enc_test_fail_next(int status) { enc::g_forced = status; }

extern "C" int enc_device_info(enc_device_info_t *out) {
    ENC_PROLOGUE();
    if (!out) return enc::fail(ENC_ERR_BAD_ARG, "enc_device_info: NULL output");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return enc::fail(ENC_ERR_LAUNCH, "enc_device_info: no CUDA device (%s)", cudaGetErrorString(e));
    cudaDeviceProp p;
    e = cudaGetDeviceProperties(&p, dev);
    if (e != cudaSuccess) return enc::fail(ENC_ERR_LAUNCH, "enc_device_info: %s", cudaGetErrorString(e));
    memset(out, 0, sizeof(*out));
    out->device = dev;
    out->sm_count = p.multiProcessorCount;
    out->cc_major = p.major;
    out->cc_minor = p.minor;
    out->max_smem_per_block = (int)p.sharedMemPerBlockOptin;
    out->l2_bytes = p.l2CacheSize;
    out->global_mem = p.totalGlobalMem;
    strncpy(out->name, p.name, sizeof(out->name) - 1);
    return ENC_OK;
}

extern "C" int enc_num_variants(int kernel) {
    switch (kernel) {
        case ENC_K_SOFTMAX: case ENC_K_LAYERNORM: case ENC_K_RMSNORM: return enc::row_variants();
        case ENC_K_GELU: return enc::gelu_variants();
        case ENC_K_HISTOGRAM: return enc::hist_variants();
        case ENC_K_CUMSUM: return enc::scan_variants();
        case ENC_K_MATMUL: return enc::matmul_variants();
        case ENC_K_ATTENTION: return enc::attention_variants();
        case ENC_K_MATMUL_INT: return enc::int_matmul_variants();
        case ENC_K_ADD: return 1;
        default: return 0;
    }
}

extern "C" int enc_variant_info(int kernel, int variant, char *out, size_t n) {
    if (!out || n == 0) return enc::fail(ENC_ERR_BAD_ARG, "enc_variant_info: no output buffer");
    if (variant < 0 || variant >= enc_num_variants(kernel))
        return enc::fail(ENC_ERR_BAD_ARG, "enc_variant_info: kernel %d has no variant %d", kernel, variant);
    switch (kernel) {
        case ENC_K_SOFTMAX: case ENC_K_LAYERNORM: case ENC_K_RMSNORM: enc::row_variant_info(variant, out, n); break;
        case ENC_K_GELU: enc::gelu_variant_info(variant, out, n); break;
        case ENC_K_HISTOGRAM: enc::hist_variant_info(variant, out, n); break;
        case ENC_K_CUMSUM: enc::scan_variant_info(variant, out, n); break;
        case ENC_K_MATMUL: enc::matmul_variant_info(variant, out, n); break;
        case ENC_K_ATTENTION: enc::attention_variant_info(variant, out, n); break;
        case ENC_K_MATMUL_INT: enc::int_matmul_variant_info(variant, out, n); break;
        default: snprintf(out, n, "cta_threads=256 grid-stride"); break;
    }
    return ENC_OK;
}

extern "C" int enc_synchronize(void *stream) {
    ENC_PROLOGUE();
    cudaError_t e = cudaStreamSynchronize(enc::as_stream(stream));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return enc::fail(ENC_ERR_LAUNCH, "enc_synchronize: CUDA error %d (%s)", (int)e, cudaGetErrorString(e));
    }
    int dev = 0;
    cudaGetDevice(&dev);
    unsigned int *w = nullptr;
    {
        std::lock_guard<std::mutex> lock(enc::g_mu);
        if (dev >= 0 && dev < enc::MAX_DEVICES) w = enc::g_error_word[dev];
    }
    if (w) {
        unsigned int host = 0;
        e = cudaMemcpy(&host, w, sizeof(host), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return enc::fail(ENC_ERR_LAUNCH, "enc_synchronize: reading the device status word failed (%s)", cudaGetErrorString(e));
        if (host) {
            cudaMemset(w, 0, sizeof(host));
            return enc::fail(ENC_ERR_DEVICE_WAIT, "a device-side wait ran out of its iteration limit (status word %u); results of the launches since the last synchronisation are invalid", host);
        }
    }
    return ENC_OK;
}
