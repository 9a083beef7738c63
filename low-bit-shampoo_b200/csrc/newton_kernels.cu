// Inverse p-th root by the coupled Newton iteration on the tensor cores, for a whole batch of
// SPD matrices, without a host synchronisation.
//
// Reference (project paths): optimizers/matrix_functions.py:22-48 (PowerIter), :52-76
// (MatPower), :80-141 (ComputePower); callers optimizers/shampoo1.py:181-201 and
// optimizers/shampoo2.py:220-230.  Per matrix the reference runs, with two host
// synchronisations per iteration,
//     lambda_max by <= 10 power iterations;  G += ridge_eps * lambda_max * I;
//     z = (1 + p) / (2 ||G||_F);  root = z^(1/p) I;  M = z G;  err = max |M - I|
//     while err > tol and count < iter_count:
//         T = (1 + 1/p) I - M / p;  root' = root T;  M' = T^p M;  err' = max |M' - I|
//         if err' > 1.2 err: break
//         root, M, err = root', M', err'
// Here every matrix follows that rule through flags in device memory: `active` switches a
// matrix's tiles off inside the product kernels, and accepted iterates are published by
// swapping per-matrix slot numbers of ping-pong buffers, never by copying.  The products run
// on the three-plane tcgen05 kernel (fp32-level accuracy), each epilogue writing the planes the
// next product reads; the epilogue of T^p M also writes the next T and reduces max |M' - I|.
#include "qt_common.cuh"
#include <math_constants.h>

namespace qt {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Block-wide sum of one double per thread (1024 threads); result valid in every thread.
__device__ __forceinline__ double block_sum(double v, double *scratch /*[32]*/) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();                                       // scratch may still be read from a previous call
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
    const int warps = blockDim.x >> 5;
    for (int i = 0; i < warps; ++i) t += scratch[i];
    return t;
}

// One CTA per matrix.  Power iteration exactly as PowerIter states it (normalise, multiply,
// Rayleigh quotient, stop when it moves by <= tol or after max_iters), then - if ridge_eps >= 0 -
// the ridge ridge_eps * lambda_max is added to the diagonal IN PLACE (the reference mutates its
// argument too, matrix_functions.py:112) and the Frobenius norm of the result is written.
__global__ void __launch_bounds__(1024, 1)
k_power_iter(float *__restrict__ Gbase, long long strideG, int n, const float *__restrict__ v0, float tol, int max_iters,
             float ridge_eps, float *__restrict__ max_ev, float *__restrict__ fro, int *__restrict__ iters_out,
             float *__restrict__ vec_out) {
    extern __shared__ float pw_sm[];
    float *v = pw_sm, *y = pw_sm + n;
    __shared__ double red[32];
    float *G = Gbase + (long long)blockIdx.x * strideG;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    for (int i = tid; i < n; i += blockDim.x) v[i] = v0[(long long)blockIdx.x * n + i];
    __syncthreads();
    const bool vec = (n & 3) == 0 && ((reinterpret_cast<uintptr_t>(G) & 15) == 0);
    float sval = 0.0f, err = 1.0f;
    int it = 0;
    while (err > tol && it < max_iters) {
        double ss = 0.0;
        for (int i = tid; i < n; i += blockDim.x) ss += (double)v[i] * (double)v[i];
        const float nrm = (float)sqrt(block_sum(ss, red));
        for (int i = tid; i < n; i += blockDim.x) v[i] = v[i] / nrm;
        __syncthreads();
        for (int r = warp; r < n; r += warps) {
            const float *row = G + (long long)r * n;
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
            if (vec) {
                for (int c = lane * 4; c < n; c += 128) {
                    const float4 g = *reinterpret_cast<const float4 *>(row + c);
                    a0 = fmaf(g.x, v[c], a0); a1 = fmaf(g.y, v[c + 1], a1);
                    a2 = fmaf(g.z, v[c + 2], a2); a3 = fmaf(g.w, v[c + 3], a3);
                }
            } else {
                for (int c = lane; c < n; c += 32) a0 = fmaf(row[c], v[c], a0);
            }
            const float d = warp_sum_f((a0 + a1) + (a2 + a3));
            if (lane == 0) y[r] = d;
        }
        __syncthreads();
        double dot = 0.0;
        for (int i = tid; i < n; i += blockDim.x) dot += (double)v[i] * (double)y[i];
        const float s = (float)block_sum(dot, red);
        err = fabsf(s - sval);
        sval = s;
        for (int i = tid; i < n; i += blockDim.x) v[i] = y[i];
        __syncthreads();
        ++it;
    }
    if (tid == 0) {
        max_ev[blockIdx.x] = sval;
        if (iters_out) iters_out[blockIdx.x] = it;
    }
    if (vec_out)
        for (int i = tid; i < n; i += blockDim.x) vec_out[(long long)blockIdx.x * n + i] = v[i];
    if (ridge_eps < 0.0f || fro == nullptr) return;
    const float ridge = ridge_eps * sval;
    for (int r = tid; r < n; r += blockDim.x) G[(long long)r * n + r] += ridge;
    __syncthreads();
    double sq = 0.0;
    for (int r = warp; r < n; r += warps) {
        const float *row = G + (long long)r * n;
        float a0 = 0.0f;
        for (int c = lane; c < n; c += 32) a0 = fmaf(row[c], row[c], a0);
        sq += (double)a0;
    }
    const double total = block_sum(sq, red);
    if (tid == 0) fro[blockIdx.x] = (float)sqrt(total);
}

__device__ __forceinline__ void split3_store(float x, __nv_bfloat16 *hi, __nv_bfloat16 *mid, __nv_bfloat16 *lo, long long o) {
    const __nv_bfloat16 h = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(h);
    const __nv_bfloat16 m = __float2bfloat16_rn(r1);
    hi[o] = h; mid[o] = m; lo[o] = __float2bfloat16_rn(r1 - __bfloat162float(m));
}

// Start of the iteration (matrix_functions.py:113-128): z = (1 + p) / (2 fro), M = z G,
// T = (1 + 1/p) I - M / p, root = z^(1/p) I, all as three-plane operands; max |M - I| is combined
// into err0 with an atomic maximum.  Planes: entry b of storages with `stride` elements per
// matrix and row pitch ld; G: n x n fp32, contiguous rows.
__global__ void __launch_bounds__(256)
k_newton_prepare(const float *__restrict__ Gbase, long long strideG, int n, const float *__restrict__ fro, float pf,
                 __nv_bfloat16 *Mh, __nv_bfloat16 *Mm, __nv_bfloat16 *Ml,
                 __nv_bfloat16 *Th, __nv_bfloat16 *Tm, __nv_bfloat16 *Tl,
                 __nv_bfloat16 *Rh, __nv_bfloat16 *Rm, __nv_bfloat16 *Rl,
                 long long ld, long long stride, float *__restrict__ err0) {
    const int b = blockIdx.y;
    const float *G = Gbase + (long long)b * strideG;
    const float z = (1.0f + pf) / (2.0f * fro[b]);
    const float r0 = powf(z, 1.0f / pf);
    const float alpha = -1.0f / pf;
    const long long base = (long long)b * stride;
    float dev = 0.0f;
    const long long total = (long long)n * n;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(e / n), c = (int)(e - (long long)r * n);
        const float m = G[e] * z;
        const float id = r == c ? 1.0f : 0.0f;
        const long long o = base + (long long)r * ld + c;
        split3_store(m, Mh, Mm, Ml, o);
        split3_store((1.0f - alpha) * id + alpha * m, Th, Tm, Tl, o);
        split3_store(r0 * id, Rh, Rm, Rl, o);
        float a = fabsf(m - id);
        if (!(a <= 3.0e38f)) a = CUDART_INF_F;
        dev = fmaxf(dev, a);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dev = fmaxf(dev, __shfl_xor_sync(0xffffffffu, dev, off));
    if ((threadIdx.x & 31) == 0 && dev > 0.0f) atomicMax(reinterpret_cast<int *>(err0 + b), __float_as_int(dev));
}

// Per-matrix bookkeeping between iterations (one thread per matrix).
//   init: err <- err_new (the start error), slots to their first halves, active = err > tol.
//   step: the reference's acceptance rule; an accepted iterate is published by swapping slots.
__global__ void k_newton_update(int batch, int init, float tol, float *__restrict__ err, float *__restrict__ err_new,
                                int *__restrict__ active, int *__restrict__ curM, int *__restrict__ othM,
                                int *__restrict__ curR, int *__restrict__ othR, int *__restrict__ iters) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    if (init) {
        err[b] = err_new[b];
        curM[b] = b; othM[b] = b + batch; curR[b] = b; othR[b] = b + batch;
        iters[b] = 0;
        active[b] = err[b] > tol ? 1 : 0;
    } else if (active[b]) {
        const float e_new = err_new[b], e_old = err[b];
        const bool accept = !(e_new > e_old * 1.2f);
        if (accept) {
            const int m = curM[b]; curM[b] = othM[b]; othM[b] = m;
            const int r = curR[b]; curR[b] = othR[b]; othR[b] = r;
            err[b] = e_new;
            iters[b] += 1;
        }
        active[b] = (accept && e_new > tol) ? 1 : 0;
    }
    err_new[b] = 0.0f;
}

// root (fp32, n x n contiguous) <- hi + mid + lo of the current root slot of every matrix.
__global__ void __launch_bounds__(256)
k_newton_finish(const __nv_bfloat16 *__restrict__ Rh, const __nv_bfloat16 *__restrict__ Rm, const __nv_bfloat16 *__restrict__ Rl,
                long long ld, long long stride, const int *__restrict__ curR, int n, float *__restrict__ out, long long strideOut) {
    const int b = blockIdx.y;
    const long long base = (long long)curR[b] * stride;
    float *O = out + (long long)b * strideOut;
    const long long total = (long long)n * n;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(e / n), c = (int)(e - (long long)r * n);
        const long long o = base + (long long)r * ld + c;
        O[e] = (__bfloat162float(Rh[o]) + __bfloat162float(Rm[o])) + __bfloat162float(Rl[o]);
    }
}

int launch_power_iter(float *G, long long strideG, int n, int batch, const float *v0, float tol, int max_iters, float ridge_eps,
                      float *max_ev, float *fro, int *iters, float *vec_out, cudaStream_t s) {
    if (n <= 0 || batch < 0 || !G || !v0 || !max_ev || max_iters < 0) return record(QT_ERR_ARG);
    if (batch == 0) return record(QT_OK);
    const size_t smem = sizeof(float) * 2 * (size_t)n;
    if (smem > 200 * 1024) return record(QT_ERR_UNSUPPORTED);
    static PerDeviceOnce attr;
    const int dev = current_device();
    if (attr.pending(dev)) {
        if (cudaFuncSetAttribute(k_power_iter, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return record(QT_ERR_LAUNCH);
        attr.mark(dev);
    }
    k_power_iter<<<batch, 1024, smem, s>>>(G, strideG, n, v0, tol, max_iters, ridge_eps, max_ev, fro, iters, vec_out);
    count_launch(1);
    return check_launch();
}

static inline long long pitch16(long long cols) { return (cols + 15) / 16 * 16; }

// Workspace layout (bytes), shared by the size query and the driver.
struct NewtonLayout {
    long long ld, stride;                  // plane pitch and elements per matrix
    size_t planes_off[7];                  // M (2B entries), T (B), R (2B), S1 (B), S2 (B): start of plane group g
    size_t floats_off, ints_off, total;
};
static NewtonLayout newton_layout(int n, int batch) {
    NewtonLayout L;
    L.ld = pitch16(n);
    L.stride = (long long)n * L.ld;
    const size_t per = (size_t)L.stride * 2;               // bytes of one plane of one matrix
    size_t off = 0;
    const int entries[5] = {2 * batch, batch, 2 * batch, batch, batch};
    for (int g = 0; g < 5; ++g) { L.planes_off[g] = off; off += 3 * per * (size_t)entries[g]; off = (off + 255) & ~(size_t)255; }
    L.floats_off = off; off += sizeof(float) * 4 * (size_t)batch; off = (off + 255) & ~(size_t)255;
    L.ints_off = off; off += sizeof(int) * 6 * (size_t)batch; off = (off + 255) & ~(size_t)255;
    L.total = off;
    return L;
}

size_t inverse_root_workspace_bytes(int n, int batch) {
    if (n <= 0 || batch <= 0) return 0;
    return newton_layout(n, batch).total;
}

// Declared in gemm_tcgen05.cu: one three-plane product with the optional extras.
int launch_newton_product(void *const A[3], const int *a_slot, int a_entries,
                          void *const B[3], const int *b_slot, int b_entries,
                          void *const P[3], const int *d_slot, void *const T[3], float t_c0, float t_c1, float *maxdev,
                          const int *active, int n, int batch, long long ld, long long stride, cudaStream_t s);

int launch_inverse_root_newton(float *G, long long strideG, int n, int batch, int p, int iter_count, float tol, float ridge_eps,
                               const float *v0, void *workspace, size_t workspace_bytes, float *out, long long strideOut,
                               float *max_ev_out, int *iters_out, cudaStream_t s) {
    if (n < 2 || batch < 0 || p < 2 || (p & (p - 1)) != 0 || p > 64 || iter_count < 0) return record(QT_ERR_UNSUPPORTED);
    if (batch == 0) return record(QT_OK);
    if (!G || !v0 || !workspace || !out) return record(QT_ERR_ARG);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return record(QT_ERR_ARG);
    const NewtonLayout L = newton_layout(n, batch);
    if (workspace_bytes < L.total) return record(QT_ERR_ARG);
    unsigned char *w = static_cast<unsigned char *>(workspace);
    const size_t per = (size_t)L.stride * 2;
    auto planes = [&](int g, int entries, void *out3[3]) {
        for (int k = 0; k < 3; ++k) out3[k] = w + L.planes_off[g] + (size_t)k * per * (size_t)entries;
    };
    void *Mp[3], *Tp[3], *Rp[3], *S1[3], *S2[3];
    planes(0, 2 * batch, Mp); planes(1, batch, Tp); planes(2, 2 * batch, Rp); planes(3, batch, S1); planes(4, batch, S2);
    float *fl = reinterpret_cast<float *>(w + L.floats_off);
    float *max_ev = fl, *fro = fl + batch, *err = fl + 2 * batch, *err_new = fl + 3 * batch;
    int *in = reinterpret_cast<int *>(w + L.ints_off);
    int *active = in, *curM = in + batch, *othM = in + 2 * batch, *curR = in + 3 * batch, *othR = in + 4 * batch, *iters = in + 5 * batch;

    int rc = launch_power_iter(G, strideG, n, batch, v0, 1e-6f, 10, ridge_eps, max_ev, fro, nullptr, nullptr, s);
    if (rc != QT_OK) return rc;
    if (cudaMemsetAsync(err_new, 0, sizeof(float) * batch, s) != cudaSuccess) return record(QT_ERR_LAUNCH);
    {
        const long long total = (long long)n * n;
        long long ctas = (total + 256 * 8 - 1) / (256 * 8);
        const long long cap = ((long long)device_sm_count() * 16 + batch - 1) / batch;
        if (ctas > cap) ctas = cap;
        if (ctas < 1) ctas = 1;
        dim3 grid((unsigned)ctas, batch);
        auto bf = [](void *q) { return static_cast<__nv_bfloat16 *>(q); };
        k_newton_prepare<<<grid, 256, 0, s>>>(G, strideG, n, fro, (float)p, bf(Mp[0]), bf(Mp[1]), bf(Mp[2]),
                                               bf(Tp[0]), bf(Tp[1]), bf(Tp[2]), bf(Rp[0]), bf(Rp[1]), bf(Rp[2]),
                                               L.ld, L.stride, err_new);
        count_launch(1);
        if ((rc = check_launch()) != QT_OK) return rc;
    }
    const unsigned ub = (unsigned)((batch + 127) / 128);
    k_newton_update<<<ub, 128, 0, s>>>(batch, 1, tol, err, err_new, active, curM, othM, curR, othR, iters);
    count_launch(1);
    if ((rc = check_launch()) != QT_OK) return rc;
    const float alpha = -1.0f / (float)p;
    void *none3[3] = {nullptr, nullptr, nullptr};
    for (int it = 0; it < iter_count; ++it) {
        // T^2 (and further squarings up to T^p) from T; the last power ends in `pw`
        void **src = Tp, **dst = S1;
        void **pw = Tp;
        for (int q = 1; q < p; q *= 2) {
            rc = launch_newton_product(src, nullptr, batch, src, nullptr, batch, dst, nullptr, none3, 0.f, 0.f, nullptr,
                                       active, n, batch, L.ld, L.stride, s);
            if (rc != QT_OK) return rc;
            pw = dst;
            src = dst;
            dst = (dst == S1) ? S2 : S1;
        }
        // root' = root T  (reads the current T: must precede the product that overwrites T)
        rc = launch_newton_product(Rp, curR, 2 * batch, Tp, nullptr, batch, Rp, othR, none3, 0.f, 0.f, nullptr,
                                   active, n, batch, L.ld, L.stride, s);
        if (rc != QT_OK) return rc;
        // M' = T^p M, next T = (1 - alpha) I + alpha M', err' = max |M' - I|
        rc = launch_newton_product(pw, nullptr, batch, Mp, curM, 2 * batch, Mp, othM, Tp, 1.0f - alpha, alpha, err_new,
                                   active, n, batch, L.ld, L.stride, s);
        if (rc != QT_OK) return rc;
        k_newton_update<<<ub, 128, 0, s>>>(batch, 0, tol, err, err_new, active, curM, othM, curR, othR, iters);
        count_launch(1);
        if ((rc = check_launch()) != QT_OK) return rc;
    }
    {
        const long long total = (long long)n * n;
        long long ctas = (total + 256 * 8 - 1) / (256 * 8);
        const long long cap = ((long long)device_sm_count() * 16 + batch - 1) / batch;
        if (ctas > cap) ctas = cap;
        if (ctas < 1) ctas = 1;
        dim3 grid((unsigned)ctas, batch);
        k_newton_finish<<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16 *>(Rp[0]), static_cast<__nv_bfloat16 *>(Rp[1]),
                                              static_cast<__nv_bfloat16 *>(Rp[2]), L.ld, L.stride, curR, n, out, strideOut);
        count_launch(1);
        if ((rc = check_launch()) != QT_OK) return rc;
    }
    if (max_ev_out && cudaMemcpyAsync(max_ev_out, max_ev, sizeof(float) * batch, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
        return record(QT_ERR_LAUNCH);
    if (iters_out && cudaMemcpyAsync(iters_out, iters, sizeof(int) * batch, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
        return record(QT_ERR_LAUNCH);
    return record(QT_OK);
}

}  // namespace qt

using namespace qt;

extern "C" {

int qt_power_iter(float *G, long long strideG, int n, int batch, const float *v0, float tol, int max_iters,
                  float *max_ev, int *iters, float *vec, void *stream) {
    return launch_power_iter(G, strideG, n, batch, v0, tol, max_iters, -1.0f, max_ev, nullptr, iters, vec, static_cast<cudaStream_t>(stream));
}

unsigned long long qt_inverse_root_newton_workspace_bytes(int n, int batch) {
    return (unsigned long long)inverse_root_workspace_bytes(n, batch);
}

int qt_inverse_root_newton(float *G, long long strideG, int n, int batch, int p, int iter_count, float tol, float ridge_eps,
                           const float *v0, void *workspace, unsigned long long workspace_bytes,
                           float *out, long long strideOut, float *max_ev, int *iters, void *stream) {
    return launch_inverse_root_newton(G, strideG, n, batch, p, iter_count, tol, ridge_eps, v0, workspace, (size_t)workspace_bytes,
                                      out, strideOut, max_ev, iters, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
