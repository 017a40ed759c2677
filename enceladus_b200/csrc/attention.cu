#include "common.cuh"
namespace enc {
int attention_variants() { return 0; }
void attention_variant_info(int, char *out, size_t n) { snprintf(out, n, "-"); }
}
extern "C" int enc_attention_fwd(const void *, const void *, const void *, void *, float *, int64_t, int64_t, int64_t, int64_t, int64_t, float, int, int, int, void *) {
    ENC_PROLOGUE();
    return enc::fail(ENC_ERR_UNSUPPORTED, "enc_attention_fwd: not built yet");
}
