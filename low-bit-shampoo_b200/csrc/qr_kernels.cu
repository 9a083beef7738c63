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
static constexpr int kQrThreads = 1024;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__global__ void __launch_bounds__(kQrThreads)
k_householder_panel(const float *__restrict__ Abase, long long strideA, int n, int j0, int w,
                    float *__restrict__ Vbase, long long strideV, float *__restrict__ Tbase, long long strideT) {
    extern __shared__ float sm[];
    const int m = n - j0;
    const int mpad = ((m + 31) & ~31) + 1;                 // odd multiple-of-32 offset: conflict-free transposes
    float *P = sm;                                         // [kPanel][mpad], column-major panel
    float *red = P + kPanel * mpad;                        // [32]
    float *tau = red + 32;                                 // [kPanel]
    float *colscale = tau + kPanel;                        // [kPanel]
    float *G = colscale + kPanel;                          // [kPanel][kPanel + 1], V^T V (strict upper part)
    float *Ts = G + kPanel * (kPanel + 1);                 // [kPanel][kPanel + 1]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = kQrThreads >> 5;
    const float *A = Abase + (long long)blockIdx.x * strideA + (long long)j0 * n + j0;

    for (int r = warp; r < m; r += nwarps)
        P[lane * mpad + r] = (lane < w) ? A[(long long)r * n + lane] : 0.0f;
    for (int i = tid; i < kPanel * (kPanel + 1); i += kQrThreads) { G[i] = 0.0f; Ts[i] = 0.0f; }
    __syncthreads();

    // sum of squares below the diagonal of column 0; later columns get theirs from the warp
    // that updates them (one block-wide barrier per column step)
    float *sig = red;                                      // sig[0..1]: double-buffered sigma
    {
        float s0 = 0.0f;
        for (int r = 1 + tid; r < m; r += kQrThreads) { float v = P[r]; s0 = fmaf(v, v, s0); }
        s0 = warp_sum(s0);
        if (lane == 0) G[warp] = s0;                       // G is free until the Gram step
        __syncthreads();
        if (tid == 0) {
            float t = 0.0f;
            for (int k = 0; k < nwarps; ++k) t += G[k];
            sig[0] = t;
        }
        __syncthreads();
        if (tid < nwarps) G[tid] = 0.0f;
    }
    for (int c = 0; c < w; ++c) {
        float *x = P + c * mpad;
        const float sigma = sig[c & 1];
        const float alpha = x[c];
        float tc = 0.0f, scale = 0.0f;
        if (sigma != 0.0f) {
            const float beta = -copysignf(sqrtf(fmaf(alpha, alpha, sigma)), alpha);
            tc = (beta - alpha) / beta;
            scale = 1.0f / (alpha - beta);
        }
        if (tid == 0) { tau[c] = tc; colscale[c] = scale; }
        // apply H_c = I - tau v v^T to the remaining panel columns (v = [1; scale * x_below])
        for (int cp = c + 1 + warp; cp < w; cp += nwarps) {
            float *y = P + cp * mpad;
            float d = 0.0f;
            for (int r = c + 1 + lane; r < m; r += 32) d = fmaf(x[r], y[r], d);
            d = warp_sum(d);
            const float f = tc * fmaf(scale, d, y[c]);
            __syncwarp();
            if (lane == 0) y[c] -= f;
            const float g = f * scale;
            float s2 = 0.0f;
            for (int r = c + 1 + lane; r < m; r += 32) {
                const float yn = fmaf(-g, x[r], y[r]);
                y[r] = yn;
                if (r > c + 1) s2 = fmaf(yn, yn, s2);
            }
            if (cp == c + 1) {                             // next pivot column: publish its sigma
                s2 = warp_sum(s2);
                if (lane == 0) sig[(c + 1) & 1] = s2;
            }
        }
        __syncthreads();
    }
    // x_below becomes v_below = scale * x_below
    for (int c = warp; c < w; c += nwarps) {
        float *x = P + c * mpad;
        const float scale = colscale[c];
        for (int r = c + 1 + lane; r < m; r += 32) x[r] *= scale;
    }
    __syncthreads();

    // G[i][j] = v_i . v_j for i < j
    int pair = 0;
    for (int j = 1; j < w; ++j) {
        for (int i = 0; i < j; ++i, ++pair) {
            if (pair % nwarps != warp) continue;
            const float *vi = P + i * mpad, *vj = P + j * mpad;
            float d = 0.0f;
            for (int r = j + 1 + lane; r < m; r += 32) d = fmaf(vi[r], vj[r], d);
            d = warp_sum(d);
            if (lane == 0) G[i * (kPanel + 1) + j] = d + vi[j];           // row j: v_j = 1, v_i = P[i][j]
        }
    }
    __syncthreads();
    if (warp == 0) {
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
    __syncthreads();

    float *V = Vbase + (long long)blockIdx.x * strideV + (long long)j0 * n + j0;
    for (int r = warp; r < m; r += nwarps)
        if (lane < w) V[(long long)r * n + lane] = (r < lane) ? 0.0f : (r == lane ? 1.0f : P[lane * mpad + r]);
    float *T = Tbase + (long long)blockIdx.x * strideT;
    for (int i = tid; i < kPanel * kPanel; i += kQrThreads) T[i] = Ts[(i / kPanel) * (kPanel + 1) + (i % kPanel)];
}

int launch_householder_panel(const float *A, long long strideA, int n, int count, int j0, int w,
                             float *V, long long strideV, float *T, long long strideT, cudaStream_t s) {
    if (n <= 0 || count < 0 || j0 < 0 || j0 >= n || w <= 0 || w > kPanel || j0 + w > n) return record(QT_ERR_ARG);
    if (!A || !V || !T) return record(QT_ERR_ARG);
    if (count == 0) return record(QT_OK);
    const int m = n - j0;
    const int mpad = ((m + 31) & ~31) + 1;
    const size_t smem = sizeof(float) * ((size_t)kPanel * mpad + 32 + 2 * kPanel + 2 * kPanel * (kPanel + 1));
    if (smem > 227 * 1024) return record(QT_ERR_UNSUPPORTED);
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(k_householder_panel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
            return record(QT_ERR_LAUNCH);
        attr_set = true;
    }
    k_householder_panel<<<count, kQrThreads, smem, s>>>(A, strideA, n, j0, w, V, strideV, T, strideT);
    count_launch(1);
    return check_launch();
}

}  // namespace qt
