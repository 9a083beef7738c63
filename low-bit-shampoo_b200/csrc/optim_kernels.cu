// Fused AdamW tail of the Shampoo step over a list of tensors (one launch for all parameters).
//
// Per element, in the reference's order (optimizers/shampoo2.py:441 and :457-466):
//     p   <- p * (1 - lr * weight_decay)
//     m   <- beta1 * m + (1 - beta1) * d
//     v   <- beta2 * v + (1 - beta2) * d * d
//     p   <- p - lr / (1 - beta1^t) * m / (sqrt(v) / sqrt(1 - beta2^t) + eps)
// where d is the (preconditioned, grafted) direction.  The reference issues these as ten
// tensor-wide operations per parameter (104 bytes of traffic per element); here every element is
// read and written once (28 bytes).  HBM-bound, no tensor cores.
//
// The tensors are described by device-resident tables (pointers and sizes per tensor, and a
// (tensor, chunk) pair per CTA), built once by the caller; the three step-dependent scalars are
// read from device memory so that a captured CUDA graph can be replayed with new values.
#include "qt_common.cuh"

namespace qt {

static constexpr int kTailThreads = 256;

__global__ void __launch_bounds__(kTailThreads)
k_adamw_tail(const long long *__restrict__ p_ptrs, const long long *__restrict__ d_ptrs,
             const long long *__restrict__ m_ptrs, const long long *__restrict__ v_ptrs,
             const long long *__restrict__ numels, const int *__restrict__ chunk_tensor,
             const int *__restrict__ chunk_index, int chunk_elems, const float *__restrict__ scalars,
             float beta1, float beta2, float a1, float a2, float eps) {
    const int t = chunk_tensor[blockIdx.x];
    const long long n = numels[t];
    const long long begin = (long long)chunk_index[blockIdx.x] * chunk_elems;
    const long long end = begin + chunk_elems < n ? begin + chunk_elems : n;
    float *p = reinterpret_cast<float *>(p_ptrs[t]);
    const float *d = reinterpret_cast<const float *>(d_ptrs[t]);
    float *m = reinterpret_cast<float *>(m_ptrs[t]);
    float *v = reinterpret_cast<float *>(v_ptrs[t]);
    const float c0 = scalars[0], c1 = scalars[1], c2 = scalars[2];   // 1/sqrt(1-beta2^t), -lr/(1-beta1^t), 1-lr*wd
    auto update = [&](float &pp, float dd, float &mm, float &vv) {
        const float p1 = pp * c2;
        mm = fmaf(a1, dd, mm * beta1);
        vv = fmaf(a2 * dd, dd, vv * beta2);
        const float denom = sqrtf(vv) * c0 + eps;
        pp = fmaf(c1, mm / denom, p1);
    };
    const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(m) |
                       reinterpret_cast<uintptr_t>(v)) & 15) == 0;       // chunk_elems is a multiple of 4
    if (vec) {
        const long long end4 = begin + ((end - begin) & ~3ll);
        for (long long i = begin + 4ll * threadIdx.x; i < end4; i += 4ll * kTailThreads) {
            float4 P = *reinterpret_cast<float4 *>(p + i), M = *reinterpret_cast<float4 *>(m + i), V = *reinterpret_cast<float4 *>(v + i);
            const float4 D = __ldg(reinterpret_cast<const float4 *>(d + i));
            update(P.x, D.x, M.x, V.x); update(P.y, D.y, M.y, V.y); update(P.z, D.z, M.z, V.z); update(P.w, D.w, M.w, V.w);
            *reinterpret_cast<float4 *>(p + i) = P;
            *reinterpret_cast<float4 *>(m + i) = M;
            *reinterpret_cast<float4 *>(v + i) = V;
        }
        for (long long i = end4 + threadIdx.x; i < end; i += kTailThreads) update(p[i], d[i], m[i], v[i]);
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kTailThreads) update(p[i], d[i], m[i], v[i]);
    }
}

int launch_adamw_tail(const long long *p_ptrs, const long long *d_ptrs, const long long *m_ptrs, const long long *v_ptrs,
                      const long long *numels, const int *chunk_tensor, const int *chunk_index, int num_chunks,
                      int chunk_elems, const float *scalars, float beta1, float beta2, float a1, float a2, float eps, cudaStream_t s) {
    if (num_chunks < 0 || chunk_elems <= 0 || chunk_elems % 4) return record(QT_ERR_ARG);
    if (num_chunks == 0) return record(QT_OK);
    if (!p_ptrs || !d_ptrs || !m_ptrs || !v_ptrs || !numels || !chunk_tensor || !chunk_index || !scalars) return record(QT_ERR_ARG);
    k_adamw_tail<<<num_chunks, kTailThreads, 0, s>>>(p_ptrs, d_ptrs, m_ptrs, v_ptrs, numels, chunk_tensor, chunk_index,
                                                     chunk_elems, scalars, beta1, beta2, a1, a2, eps);
    count_launch(1);
    return check_launch();
}

// Column-wise dot products of two batches of row-major matrices: out[b][j] = sum_i A[b][i][j] B[b][i][j]
// - the Rayleigh quotients diag(V^T (L V)) of the eigenbasis refresh (qtensor/utils.py:158 forms the
// whole product V^T L V and takes its diagonal).  One CTA per (32 columns, matrix): thread (ty, tx)
// walks rows ty, ty+32, .. of column tx with four accumulators, then the 32 partial sums of a column
// are added in a fixed tree.  The summation order depends on the matrix shape only, never on the
// batch: a matrix gets the same bits alone, in a shard or in the full class (a library reduction
// over the same data picks its launch configuration - and with it the order - from the batch size).
__global__ void __launch_bounds__(1024)
k_column_dot(const float *__restrict__ Abase, const float *__restrict__ Bbase, long long ld, long long stride,
             int rows, int cols, float *__restrict__ out, long long stride_out) {
    __shared__ float part[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int j = blockIdx.x * 32 + tx;
    const float *A = Abase + (long long)blockIdx.y * stride, *B = Bbase + (long long)blockIdx.y * stride;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (j < cols) {
        int k = 0;
        for (int i = ty; i < rows; i += 32, ++k)
            acc[k & 3] = fmaf(__ldg(A + (long long)i * ld + j), __ldg(B + (long long)i * ld + j), acc[k & 3]);
    }
    part[ty][tx] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    __syncthreads();
    if (ty == 0 && j < cols) {
        float s[32];
#pragma unroll
        for (int q = 0; q < 32; ++q) s[q] = part[q][tx];
#pragma unroll
        for (int w = 16; w > 0; w >>= 1)
#pragma unroll
            for (int q = 0; q < w; ++q) s[q] += s[q + w];
        out[(long long)blockIdx.y * stride_out + j] = s[0];
    }
}

int launch_column_dot(const float *A, const float *B, long long ld, long long stride, int rows, int cols, int batch,
                      float *out, long long stride_out, cudaStream_t s) {
    if (rows < 0 || cols < 0 || batch < 0 || batch > 65535 || ld < cols) return record(QT_ERR_ARG);
    if (cols == 0 || batch == 0) return record(QT_OK);
    if (!A || !B || !out) return record(QT_ERR_ARG);
    dim3 grid((cols + 31) / 32, batch);
    k_column_dot<<<grid, 1024, 0, s>>>(A, B, ld, stride, rows, cols, out, stride_out);
    count_launch(1);
    return check_launch();
}

}  // namespace qt

extern "C" int qt_column_dot(const float *A, const float *B, long long ld, long long stride, int rows, int cols, int batch,
                             float *out, long long stride_out, void *stream) {
    return qt::launch_column_dot(A, B, ld, stride, rows, cols, batch, out, stride_out, static_cast<cudaStream_t>(stream));
}

extern "C" int qt_adamw_tail(const long long *p_ptrs, const long long *d_ptrs, const long long *m_ptrs, const long long *v_ptrs,
                             const long long *numels, const int *chunk_tensor, const int *chunk_index, int num_chunks,
                             int chunk_elems, const float *scalars, float beta1, float beta2, float one_minus_beta1,
                             float one_minus_beta2, float eps, void *stream) {
    return qt::launch_adamw_tail(p_ptrs, d_ptrs, m_ptrs, v_ptrs, numels, chunk_tensor, chunk_index, num_chunks, chunk_elems,
                                 scalars, beta1, beta2, one_minus_beta1, one_minus_beta2, eps, static_cast<cudaStream_t>(stream));
}
