// Batched Householder panel factorisation for the eigenbasis refresh of the statistics.
//
// The reference orthonormalises L V with torch.linalg.qr (reference project path
// qtensor/utils.py:157), i.e. one cuSOLVER geqrf + orgqr per matrix.  Here a whole order
// class is factorised together: this kernel factors one 32-column panel of every matrix
// of the batch (one CTA per matrix, the panel resident in shared memory) and emits the
// Householder vectors V (unit lower trapezoidal, explicit zeros and ones) and the
// triangular factor T of the compact-WY form  H_1 .. H_w = I - V T V^T.  The trailing
// update and the accumulation of Q are batched matrix products issued by the caller.
//
// Conventions are LAPACK's (slarfg / slarft, forward, columnwise): beta = -sign(alpha)
// * ||x||, tau = (beta - alpha) / beta, v = x / (alpha - beta) with v_0 = 1; a column
// that is already zero below the diagonal gets tau = 0.
#include "qt_common.cuh"

namespace qt {

static constexpr int kPanel = 32;
static constexpr int kQrThreads = 1024;                    // one warp per panel column
static constexpr int kMaxRowsPerLane = 38;                 // panel rows <= 32 * 38 = 1216

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Register-resident panel: warp c owns column c, lane l holds rows l, l+32, ... of it (RPL
// values) for the whole factorisation.  Per column step the pivot warp builds its Householder
// vector from registers and publishes it once through a double-buffered shared-memory vector;
// the warps to its right apply the reflector to their own registers, the warps to its left
// (already final) take the dot product v_i . v_c needed for the triangular factor T.  Shared
// memory traffic per step is one vector write and one read per warp, one barrier per step.
template <int RPL>
__global__ void __launch_bounds__(kQrThreads, 1)
k_householder_panel(const float *__restrict__ Abase, long long strideA, int n, int j0, int w,
                    float *__restrict__ Vbase, long long strideV, float *__restrict__ Tbase, long long strideT) {
    extern __shared__ float sm[];
    const int m = n - j0;
    float *P = sm;                                         // [m][33] staging for coalesced global access
    float *vb = P + ((m * 33 + 31) & ~31);                 // [2][RPL * 32] published Householder vector
    float *G = vb + 2 * RPL * 32;                          // [32][33]  v_i . v_j, i < j
    float *Ts = G + kPanel * (kPanel + 1);                 // [32][33]
    float *tau = Ts + kPanel * (kPanel + 1);               // [32]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *A = Abase + (long long)blockIdx.x * strideA + (long long)j0 * n + j0;

    for (int r = warp; r < m; r += 32) P[r * 33 + lane] = (lane < w) ? A[(long long)r * n + lane] : 0.0f;
    for (int i = tid; i < 2 * kPanel * (kPanel + 1); i += kQrThreads) G[i] = 0.0f;   // G and Ts are adjacent
    __syncthreads();
    float col[RPL];
#pragma unroll
    for (int k = 0; k < RPL; ++k) {
        const int r = lane + 32 * k;
        col[k] = (r < m) ? P[r * 33 + warp] : 0.0f;
    }

    for (int c = 0; c < w; ++c) {
        float *vbuf = vb + (c & 1) * (RPL * 32);
        if (warp == c) {
            float s = 0.0f;
#pragma unroll
            for (int k = 0; k < RPL; ++k) s = (lane + 32 * k > c) ? fmaf(col[k], col[k], s) : s;
            const float sigma = warp_sum(s);
            const float alpha = __shfl_sync(0xffffffffu, col[0], c);      // row c lives in lane c, slot 0
            float tc = 0.0f, scale = 0.0f;
            if (sigma != 0.0f) {
                const float beta = -copysignf(sqrtf(fmaf(alpha, alpha, sigma)), alpha);
                tc = (beta - alpha) / beta;
                scale = 1.0f / (alpha - beta);
            }
#pragma unroll
            for (int k = 0; k < RPL; ++k) {
                const int r = lane + 32 * k;
                const float v = (r > c) ? col[k] * scale : (r == c ? 1.0f : 0.0f);
                col[k] = v;                                 // the column now holds v_c (zeros above, one on the diagonal)
                vbuf[k * 32 + lane] = v;
            }
            if (lane == 0) tau[c] = tc;
        }
        __syncthreads();
        if (warp != c && warp < w) {
            float d = 0.0f;
#pragma unroll
            for (int k = 0; k < RPL; ++k) d = fmaf(vbuf[k * 32 + lane], col[k], d);
            d = warp_sum(d);
            if (warp > c) {                                 // apply H_c = I - tau v v^T to this column
                const float f = tau[c] * d;
#pragma unroll
                for (int k = 0; k < RPL; ++k) col[k] = fmaf(-f, vbuf[k * 32 + lane], col[k]);
            } else if (lane == 0) {
                G[warp * (kPanel + 1) + c] = d;             // v_warp . v_c
            }
        }
    }
    __syncthreads();
    if (warp == 0) {                                        // LAPACK slarft, forward / columnwise
        for (int i = 0; i < w; ++i) {
            const float ti = tau[i];
            if (lane == i) Ts[i * (kPanel + 1) + i] = ti;
            if (lane < i) {
                float acc = 0.0f;
                for (int l = lane; l < i; ++l) acc = fmaf(Ts[lane * (kPanel + 1) + l], G[l * (kPanel + 1) + i], acc);
                Ts[lane * (kPanel + 1) + i] = -ti * acc;
            }
            __syncwarp();
        }
    }
#pragma unroll
    for (int k = 0; k < RPL; ++k) {
        const int r = lane + 32 * k;
        if (r < m) P[r * 33 + warp] = col[k];
    }
    __syncthreads();
    float *V = Vbase + (long long)blockIdx.x * strideV + (long long)j0 * n + j0;
    for (int r = warp; r < m; r += 32)
        if (lane < w) V[(long long)r * n + lane] = P[r * 33 + lane];
    float *T = Tbase + (long long)blockIdx.x * strideT;
    for (int i = tid; i < kPanel * kPanel; i += kQrThreads) T[i] = Ts[(i / kPanel) * (kPanel + 1) + (i % kPanel)];
}

template <int RPL>
static int launch_panel_rpl(const float *A, long long strideA, int n, int count, int j0, int w,
                            float *V, long long strideV, float *T, long long strideT, cudaStream_t s) {
    const int m = n - j0;
    const size_t smem = sizeof(float) * ((size_t)((m * 33 + 31) & ~31) + 2 * RPL * 32 + 2 * kPanel * (kPanel + 1) + kPanel);
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(k_householder_panel<RPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
            return record(QT_ERR_LAUNCH);
        attr_set = true;
    }
    if (smem > 227 * 1024) return record(QT_ERR_UNSUPPORTED);
    k_householder_panel<RPL><<<count, kQrThreads, smem, s>>>(A, strideA, n, j0, w, V, strideV, T, strideT);
    count_launch(1);
    return check_launch();
}

int launch_householder_panel(const float *A, long long strideA, int n, int count, int j0, int w,
                             float *V, long long strideV, float *T, long long strideT, cudaStream_t s) {
    if (n <= 0 || count < 0 || j0 < 0 || j0 >= n || w <= 0 || w > kPanel || j0 + w > n) return record(QT_ERR_ARG);
    if (!A || !V || !T) return record(QT_ERR_ARG);
    if (count == 0) return record(QT_OK);
    const int rows_per_lane = (n - j0 + 31) / 32;
    if (rows_per_lane > kMaxRowsPerLane) return record(QT_ERR_UNSUPPORTED);
#define QT_PANEL(R) return launch_panel_rpl<R>(A, strideA, n, count, j0, w, V, strideV, T, strideT, s)
    if (rows_per_lane <= 6) QT_PANEL(6);
    if (rows_per_lane <= 12) QT_PANEL(12);
    if (rows_per_lane <= 20) QT_PANEL(20);
    if (rows_per_lane <= 28) QT_PANEL(28);
    QT_PANEL(38);
#undef QT_PANEL
}

}  // namespace qt
