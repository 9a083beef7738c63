// Shared declarations of libqtensor_b200: status codes, stream / error bookkeeping and
// the launcher prototypes that abi.cu forwards to.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/qtensor_b200.h"

namespace qt {

// Thread-local state behind qt_set_stream / qt_last_error.
cudaStream_t current_stream();
void set_current_stream(cudaStream_t s);
int record(int status);          // stores status as this thread's last error and returns it
void count_launch(int n);        // adds n to the process-wide kernel launch counter
int check_launch();              // cudaGetLastError -> QT_OK / QT_ERR_LAUNCH (recorded)

// Per-device bookkeeping: function attributes (cudaFuncSetAttribute) and the SM count belong to
// one device, and a process may drive several.  Ordinals at or above kMaxDevices are refused.
static constexpr int kMaxDevices = 64;
int current_device();            // ordinal of the calling thread's current device, or -1
int device_sm_count();           // SM count of the current device (cached per device; 148 if unknown)
// One flag per device.  pending() is true until mark() has been called for that device; a
// race between two first callers only repeats an idempotent set-up.
struct PerDeviceOnce {
    volatile unsigned char done[kMaxDevices];
    bool pending(int dev) const { return dev < 0 || dev >= kMaxDevices || !done[dev]; }
    void mark(int dev) { if (dev >= 0 && dev < kMaxDevices) done[dev] = 1; }
};

inline bool valid_blocksize(int bs) {
    return bs == 64 || bs == 128 || bs == 256 || bs == 512 || bs == 1024 || bs == 2048;
}

struct QuantArgs {
    const void *A; int a_dtype; long long strideA;          // elements
    const float *code;
    int n, count, bs, bits;
    float *absmax; long long stride_absmax;
    float *diag; long long stride_diag;                     // diag == nullptr: plain variant
    unsigned char *out; long long stride_out;               // bytes
};

struct DequantArgs {
    const unsigned char *A; long long strideA;              // bytes
    const float *code;
    int n, count, bs, bits;
    const float *absmax; long long stride_absmax;
    const float *diag; long long stride_diag;
    void *out; int out_dtype; long long stride_out;         // elements
};

int launch_merge_t(const float *G, long long ldg, long long strideG, const float *Tp, long long strideTp, int wo, int count,
                   float *T, long long strideT, cudaStream_t stream);
int launch_quantize(const QuantArgs &a, cudaStream_t stream);
int launch_dequantize(const DequantArgs &a, cudaStream_t stream);
// a.out / a.out_dtype / a.stride_out are ignored: output goes to the bf16 planes hi, lo
// amax_scratch != nullptr: scaled fp16 planes (exponents from each matrix's largest magnitude and
// `target`, written to exp_out); nullptr: plain bf16 planes.
int launch_dequantize_planes(const DequantArgs &a, const int *slots, void *hi, void *lo, long long ldp, long long strideP,
                             cudaStream_t stream, float *amax_scratch = nullptr, int target = 0, int *exp_out = nullptr);
int launch_state_exponents(const float *absmax, long long stride_absmax, int n_absmax, const float *diag, long long stride_diag,
                           int n_diag, const int *slots, int count, int target, int *exp_out, cudaStream_t stream);
int launch_selftest_division(unsigned long long seed, unsigned long long pairs, unsigned long long *mismatches_dev,
                             cudaStream_t stream);
void set_panel_pairs(int on);
int launch_householder_panel(float *A, long long strideA, int n, int count, int j0, int w,
                             float *V, long long strideV, float *T, long long strideT, cudaStream_t stream,
                             int prev_w = 0, const float *Tprev = nullptr, int block_end = 0);

}  // namespace qt
