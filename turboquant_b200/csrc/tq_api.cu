// Host-side pieces shared by the C ABI: error text, codebook constants, device queries.
#include <cmath>
#include <cstring>

#include "tq_common.cuh"

namespace tq {

char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

// Lloyd-Max centroids for N(0,1) as tabulated by the reference (turboquant/codebook.py:16-55).
// They define the storage format: a code is an index into exactly this table.
static const double kC1[2] = {-0.7978845608028654, 0.7978845608028654};
static const double kC2[4] = {-1.5104176088887660, -0.4527800398860679, 0.4527800398860679,
                              1.5104176088887660};
static const double kC3[8] = {-2.1519775207392190, -1.3439709227384000, -0.7560052489261838,
                              -0.2451209601065855, 0.2451209601065855,  0.7560052489261838,
                              1.3439709227384000,  2.1519775207392190};
const double kCentroidsN01_4bit[16] = {
    -2.7326368237440100, -2.0693470280837980, -1.6180344937899930, -1.2562490887894980,
    -0.9423683558764893, -0.6567591430551046, -0.3880823046410021, -0.1284153814744918,
    0.1284153814744918,  0.3880823046410021,  0.6567591430551046,  0.9423683558764893,
    1.2562490887894980,  1.6180344937899930,  2.0693470280837980,  2.7326368237440100};

// Products are formed in double and rounded once to fp32, as torch.tensor does with the
// python floats of codebook.py:80-90.
void host_codebook(int dim, int bits, float* centroids, float* boundaries) {
    const double* c = bits == 1 ? kC1 : bits == 2 ? kC2 : bits == 3 ? kC3 : kCentroidsN01_4bit;
    const int n = 1 << bits;
    const double scale = 1.0 / std::sqrt((double)dim);
    for (int i = 0; i < n; i++) centroids[i] = (float)(c[i] * scale);
    for (int i = 0; i + 1 < n; i++) boundaries[i] = (float)(((c[i] + c[i + 1]) / 2.0) * scale);
}

int device_sm_count(int* out) {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (dev != cached_dev) {
        TQ_CUDA(cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev));
        cached_dev = dev;
    }
    *out = cached;
    return TQ_OK;
}

int write_fault_count(int32_t* out);
int dequant_fault_count(int32_t* out);
int pages_fault_count(int32_t* out);

}  // namespace tq

extern "C" int tq_fault_counts(int32_t* counts3) {
    TQ_REQUIRE(counts3 != nullptr, TQ_ERR_INVALID, "null pointer");
    int rc = tq::write_fault_count(counts3);
    if (rc == TQ_OK) rc = tq::dequant_fault_count(counts3 + 1);
    if (rc == TQ_OK) rc = tq::pages_fault_count(counts3 + 2);
    return rc;
}

extern "C" int tq_abi_version(void) { return TQ_ABI_VERSION; }

extern "C" const char* tq_last_error(void) { return tq::error_buffer(); }

extern "C" int tq_codebook(int dim, int bits, float* centroids, float* boundaries) {
    TQ_REQUIRE(centroids && boundaries, TQ_ERR_INVALID, "null pointer");
    TQ_REQUIRE(bits >= 1 && bits <= 4 && dim >= 1, TQ_ERR_INVALID, "bits must be 1..4, dim >= 1");
    tq::host_codebook(dim, bits, centroids, boundaries);
    return TQ_OK;
}
