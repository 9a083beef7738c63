// extern "C" surface of libqtensor_b200.so (declared in include/qtensor_b200.h).
// The sixteen legacy symbols mirror the reference's pythonInterface.cpp:27-52; they keep
// the void return type and record failures instead of exiting the process.
#include "qt_common.cuh"
#include <atomic>

namespace qt {

static thread_local cudaStream_t tl_stream = nullptr;
static thread_local int tl_last_error = QT_OK;

cudaStream_t current_stream() { return tl_stream; }
void set_current_stream(cudaStream_t s) { tl_stream = s; }
static std::atomic<unsigned long long> g_launches{0};
int record(int status) { tl_last_error = status; return status; }
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
int check_launch() {
    cudaError_t e = cudaGetLastError();
    return record(e == cudaSuccess ? QT_OK : QT_ERR_LAUNCH);
}

int current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return -1; }
    return dev;
}
int device_sm_count() {
    static std::atomic<int> cache[kMaxDevices];
    const int dev = current_device();
    if (dev >= 0 && dev < kMaxDevices) {
        const int c = cache[dev].load(std::memory_order_relaxed);
        if (c > 0) return c;
    }
    int n = 0;
    if (dev < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < kMaxDevices) cache[dev].store(n, std::memory_order_relaxed);
    return n;
}

static void legacy_quantize(const void *A, int dtype, const float *code, int order, float *absmax, float *diag,
                            unsigned char *out, int blocksize, int bits, bool diagreal) {
    if (diagreal && !diag) { record(QT_ERR_ARG); return; }
    QuantArgs a{A, dtype, 0, code, order, 1, blocksize, bits, absmax, 0, diagreal ? diag : nullptr, 0, out, 0};
    launch_quantize(a, tl_stream);
}
static void legacy_dequantize(const unsigned char *A, const float *code, int order, const float *absmax,
                              const float *diag, void *out, int dtype, int blocksize, int bits, bool diagreal) {
    if (diagreal && !diag) { record(QT_ERR_ARG); return; }
    DequantArgs a{A, 0, code, order, 1, blocksize, bits, absmax, 0, diagreal ? diag : nullptr, 0, out, dtype, 0};
    launch_dequantize(a, tl_stream);
}

}  // namespace qt

using namespace qt;

extern "C" {

void cquantize_blockwise_8bit_bf16(void *A, float *code, int order, float *absmax, unsigned char *out, int blocksize) { legacy_quantize(A, QT_BF16, code, order, absmax, nullptr, out, blocksize, 8, false); }
void cquantize_blockwise_8bit_fp32(float *A, float *code, int order, float *absmax, unsigned char *out, int blocksize) { legacy_quantize(A, QT_F32, code, order, absmax, nullptr, out, blocksize, 8, false); }
void cquantize_blockwise_4bit_bf16(void *A, float *code, int order, float *absmax, unsigned char *out, int blocksize) { legacy_quantize(A, QT_BF16, code, order, absmax, nullptr, out, blocksize, 4, false); }
void cquantize_blockwise_4bit_fp32(float *A, float *code, int order, float *absmax, unsigned char *out, int blocksize) { legacy_quantize(A, QT_F32, code, order, absmax, nullptr, out, blocksize, 4, false); }

void cdequantize_blockwise_8bit_bf16(unsigned char *A, float *code, int order, float *absmax, void *out, int blocksize) { legacy_dequantize(A, code, order, absmax, nullptr, out, QT_BF16, blocksize, 8, false); }
void cdequantize_blockwise_8bit_fp32(unsigned char *A, float *code, int order, float *absmax, float *out, int blocksize) { legacy_dequantize(A, code, order, absmax, nullptr, out, QT_F32, blocksize, 8, false); }
void cdequantize_blockwise_4bit_bf16(unsigned char *A, float *code, int order, float *absmax, void *out, int blocksize) { legacy_dequantize(A, code, order, absmax, nullptr, out, QT_BF16, blocksize, 4, false); }
void cdequantize_blockwise_4bit_fp32(unsigned char *A, float *code, int order, float *absmax, float *out, int blocksize) { legacy_dequantize(A, code, order, absmax, nullptr, out, QT_F32, blocksize, 4, false); }

void cquantize_blockwise_diagreal_8bit_bf16(void *A, float *code, int order, float *absmax, float *diag, unsigned char *out, int blocksize) { legacy_quantize(A, QT_BF16, code, order, absmax, diag, out, blocksize, 8, true); }
void cquantize_blockwise_diagreal_8bit_fp32(float *A, float *code, int order, float *absmax, float *diag, unsigned char *out, int blocksize) { legacy_quantize(A, QT_F32, code, order, absmax, diag, out, blocksize, 8, true); }
void cquantize_blockwise_diagreal_4bit_bf16(void *A, float *code, int order, float *absmax, float *diag, unsigned char *out, int blocksize) { legacy_quantize(A, QT_BF16, code, order, absmax, diag, out, blocksize, 4, true); }
void cquantize_blockwise_diagreal_4bit_fp32(float *A, float *code, int order, float *absmax, float *diag, unsigned char *out, int blocksize) { legacy_quantize(A, QT_F32, code, order, absmax, diag, out, blocksize, 4, true); }

void cdequantize_blockwise_diagreal_8bit_bf16(unsigned char *A, float *code, int order, float *absmax, float *diag, void *out, int blocksize) { legacy_dequantize(A, code, order, absmax, diag, out, QT_BF16, blocksize, 8, true); }
void cdequantize_blockwise_diagreal_8bit_fp32(unsigned char *A, float *code, int order, float *absmax, float *diag, float *out, int blocksize) { legacy_dequantize(A, code, order, absmax, diag, out, QT_F32, blocksize, 8, true); }
void cdequantize_blockwise_diagreal_4bit_bf16(unsigned char *A, float *code, int order, float *absmax, float *diag, void *out, int blocksize) { legacy_dequantize(A, code, order, absmax, diag, out, QT_BF16, blocksize, 4, true); }
void cdequantize_blockwise_diagreal_4bit_fp32(unsigned char *A, float *code, int order, float *absmax, float *diag, float *out, int blocksize) { legacy_dequantize(A, code, order, absmax, diag, out, QT_F32, blocksize, 4, true); }

int qt_version(void) { return 100; }
unsigned long long qt_launch_count(void) { return qt::g_launches.load(std::memory_order_relaxed); }
void qt_note_graph_replay(unsigned long long kernels) { qt::count_launch((int)kernels); }
int qt_last_error(void) { return tl_last_error; }
const char *qt_error_string(int status) {
    switch (status) {
        case QT_OK: return "ok";
        case QT_ERR_ARG: return "invalid argument (null pointer, negative size or misaligned buffer)";
        case QT_ERR_BLOCKSIZE: return "blocksize must be one of 64, 128, 256, 512, 1024, 2048";
        case QT_ERR_BITS: return "bits must be 4 or 8";
        case QT_ERR_LAUNCH: return "CUDA reported an error at kernel launch";
        case QT_ERR_DTYPE: return "dtype tag must be QT_F32 or QT_BF16";
        case QT_ERR_UNSUPPORTED: return "shape not supported by this kernel family";
        case QT_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case QT_ERR_RANGE: return "a value left the range of a scaled fp16 operand plane (operand exponents too large for the data)";
        case QT_ERR_TOO_LARGE: return "operands need more scratch than the library's fixed 16 MiB array holds";
        default: return "unknown status";
    }
}
void qt_set_stream(void *stream) { set_current_stream(static_cast<cudaStream_t>(stream)); }

int qt_quantize_blockwise(const void *A, int a_dtype, long long strideA, const float *code, int order, int count,
                          float *absmax, long long stride_absmax, float *diag, long long stride_diag,
                          unsigned char *out, long long stride_out, int blocksize, int bits, void *stream) {
    QuantArgs a{A, a_dtype, strideA, code, order, count, blocksize, bits, absmax, stride_absmax,
                diag, stride_diag, out, stride_out};
    return launch_quantize(a, static_cast<cudaStream_t>(stream));
}

int qt_dequantize_blockwise(const unsigned char *A, long long strideA, const float *code, int order, int count,
                            const float *absmax, long long stride_absmax, const float *diag, long long stride_diag,
                            void *out, int out_dtype, long long stride_out, int blocksize, int bits, void *stream) {
    DequantArgs a{A, strideA, code, order, count, blocksize, bits, absmax, stride_absmax,
                  diag, stride_diag, out, out_dtype, stride_out};
    return launch_dequantize(a, static_cast<cudaStream_t>(stream));
}

int qt_dequantize_planes(const unsigned char *A, long long strideA, const float *code, int order, int count,
                         const float *absmax, long long stride_absmax, const float *diag, long long stride_diag,
                         const int *slots, void *hi, void *lo, long long ldp, long long strideP,
                         int blocksize, int bits, void *stream) {
    DequantArgs a{A, strideA, code, order, count, blocksize, bits, absmax, stride_absmax,
                  diag, stride_diag, nullptr, QT_BF16, 0};
    return launch_dequantize_planes(a, slots, hi, lo, ldp, strideP, static_cast<cudaStream_t>(stream));
}

int qt_dequantize_planes_f16(const unsigned char *A, long long strideA, const float *code, int order, int count,
                             const float *absmax, long long stride_absmax, const float *diag, long long stride_diag,
                             const int *slots, float *amax_scratch, int target, int *exp_out,
                             void *hi, void *lo, long long ldp, long long strideP, int blocksize, int bits, void *stream) {
    if (!amax_scratch) return record(QT_ERR_ARG);
    DequantArgs a{A, strideA, code, order, count, blocksize, bits, absmax, stride_absmax,
                  diag, stride_diag, nullptr, QT_BF16, 0};
    return launch_dequantize_planes(a, slots, hi, lo, ldp, strideP, static_cast<cudaStream_t>(stream), amax_scratch, target, exp_out);
}

int qt_state_exponents(const float *absmax, long long stride_absmax, int n_absmax,
                       const float *diag, long long stride_diag, int n_diag,
                       const int *slots, int count, int target, int *exp_out, void *stream) {
    return launch_state_exponents(absmax, stride_absmax, n_absmax, diag, stride_diag, n_diag, slots, count, target, exp_out,
                                  static_cast<cudaStream_t>(stream));
}

int qt_selftest_division(unsigned long long seed, unsigned long long pairs, unsigned long long *mismatches, void *stream) {
    return launch_selftest_division(seed, pairs, mismatches, static_cast<cudaStream_t>(stream));
}

int qt_merge_t(const float *G, long long ldg, long long strideG, const float *Tp, long long strideTp, int width, int count,
               float *T, long long strideT, void *stream) {
    return launch_merge_t(G, ldg, strideG, Tp, strideTp, width, count, T, strideT, static_cast<cudaStream_t>(stream));
}

int qt_householder_panel(const float *A, long long strideA, int order, int count, int j0, int width,
                         float *V, long long strideV, float *T, long long strideT, void *stream) {
    return launch_householder_panel(const_cast<float *>(A), strideA, order, count, j0, width, V, strideV, T, strideT,
                                    static_cast<cudaStream_t>(stream));
}

int qt_householder_panel_fused(float *A, long long strideA, int order, int count, int j0, int width,
                               float *V, long long strideV, float *T, long long strideT,
                               int prev_width, const float *Tprev, int block_end, void *stream) {
    return launch_householder_panel(A, strideA, order, count, j0, width, V, strideV, T, strideT,
                                    static_cast<cudaStream_t>(stream), prev_width, Tprev, block_end);
}

void qt_panel_force_form(int form) { set_panel_pairs(form == 1 ? 0 : 1); }

}  // extern "C"
