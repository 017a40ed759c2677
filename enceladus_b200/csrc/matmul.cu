#include "common.cuh"
namespace enc {
int matmul_variants() { return 0; }
void matmul_variant_info(int, char *out, size_t n) { snprintf(out, n, "-"); }
}
extern "C" int enc_matmul(const void *, const void *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, int, int, void *) {
    ENC_PROLOGUE();
    return enc::fail(ENC_ERR_UNSUPPORTED, "enc_matmul: not built yet");
}
