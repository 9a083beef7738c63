// Blockwise low-bit quantize / dequantize of square matrices for sm_100a.
//
// Semantics follow the reference's CPU quantizer (reference project paths):
//   qtensor/functional.py:526-615 (_quantize_blockwise_cpu), :618-688
//   (_dequantize_blockwise_cpu), :703-715 (_nearest_code_indices), :718-746 (nibble
//   packing) - and replace the CUDA kernels of cudaC_python/csrc/kernels.cu:57-457.
//
// Design (HBM-bound byte work, no tensor cores):
//   * one launch covers a strided batch of same-order matrices (quantize: one resident wave
//     of CTAs striding over the blocks of the whole batch; dequantize: gridDim.y = matrix);
//   * a quantization block (64..256 elements of one row) is owned by a group of LPU
//     lanes of one warp, EPL consecutive elements per lane, loaded as 128-bit vectors;
//     the per-block absmax is a shuffle reduction inside the group;
//   * the nearest-code rule |q-c_lo| > |c_hi-q| (fp32) is monotone in q, so it is
//     replaced by 2^bits-1 exact fp32 thresholds found once per CTA by bisection over
//     float bit patterns; the code index is the number of thresholds <= q.  For 16-entry
//     codebooks a lookup table in shared memory (257 or 1025 cells of q, one 32-bit word each)
//     gives (base index, threshold) per cell so that one LDS.32 and one compare resolve an element;
//   * q = x / absmax is an IEEE-rounded fp32 division (the oracle divides);
//   * codes are packed high-nibble-first and stored as 16/32-bit words.
//   Orders that are not a multiple of 4, unaligned buffers and block sizes above 256
//   take a generic two-kernel path (absmax pass, then one thread per output byte).
#include "quant_device.cuh"
#include <cuda_fp16.h>

namespace qt {

static constexpr int kThreads = 256;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// 256-bit global accesses (sm_100): one request per lane for 32 bytes, half the L1 wavefronts of
// two 128-bit ones.  The address must be 32-byte aligned.
__device__ __forceinline__ void ldg256(const void *p, unsigned (&w)[8]) {
    asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "l"(p));
}
__device__ __forceinline__ void stg256(void *p, const float (&v)[8]) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
}
// 16 consecutive elements (64 bytes of fp32, 32 bytes of bf16) with 256-bit loads.
template <typename T>
__device__ __forceinline__ void load16_wide(const T *p, float (&x)[16]) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            unsigned w[8];
            ldg256(p + 8 * h, w);
#pragma unroll
            for (int j = 0; j < 8; ++j) x[8 * h + j] = __uint_as_float(w[j]);
        }
    } else {
        unsigned w[8];
        ldg256(p, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            x[2 * j] = __uint_as_float(w[j] << 16);
            x[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}

// Load EPL consecutive elements (EPL*sizeof(T) is 8, 16 or 32 bytes, pointer aligned to it or 16).
template <typename T, int EPL>
__device__ __forceinline__ void load_vec(const T *p, float (&x)[EPL]) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int j = 0; j < EPL; j += 4) {
            float4 v = __ldg(reinterpret_cast<const float4 *>(p + j));
            x[j] = v.x; x[j + 1] = v.y; x[j + 2] = v.z; x[j + 3] = v.w;
        }
    } else {
        if constexpr (EPL >= 8) {
#pragma unroll
            for (int h = 0; h < EPL / 8; ++h) {
                uint4 v = __ldg(reinterpret_cast<const uint4 *>(p + 8 * h));
                unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    x[8 * h + 2 * j] = __uint_as_float(w[j] << 16);
                    x[8 * h + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                }
            }
        } else {
            uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
            x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
            x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
        }
    }
}

// ------------------------------------------------------------------------------------
// Quantize, vector path.  Requires n % EPL == 0 and vector-aligned buffers.
// ------------------------------------------------------------------------------------
template <typename T, int BITS, int EPL, int LPU>
__global__ void __launch_bounds__(kThreads, 4)
k_quantize_vec(const T *__restrict__ Abase, long long strideA, const float *__restrict__ code,
               int n, int nb, int count, float *__restrict__ absmax_base, long long stride_absmax,
               float *__restrict__ diag_base, long long stride_diag,
               unsigned char *__restrict__ out_base, long long stride_out, int wide) {
    constexpr int NC = 1 << BITS;
    constexpr int BS = EPL * LPU;
    // `wide` (EPL == 16 only): every lane's 16 elements start on a 32-byte boundary
    auto load_lane = [&](const T *p, float (&dst)[EPL]) {
        if constexpr (EPL == 16) {
            if (wide) { load16_wide<T>(p, dst); return; }
        }
        load_vec<T, EPL>(p, dst);
    };
    __shared__ CodeTables<NC> tab;

    // A warp works on one block column of GW consecutive rows (a "warp unit": GW quantization
    // blocks, LPU lanes each), so the diagonal crosses only one warp unit in nb and the diagonal
    // side channel costs nothing elsewhere.  Warp units are numbered across the whole batch
    // (matrix, row band, block) and the grid is one resident wave striding over them: the tables
    // are built once per resident CTA and no second wave of CTAs trails behind.
    constexpr int GW = 32 / LPU;
    const int bands = (n + GW - 1) / GW;
    const int wunits = bands * nb;                          // per matrix
    const int total = wunits * count;                       // launcher keeps this below 2^31
    const int SW = gridDim.x * (kThreads / 32);             // warps striding over the batch
    const int lane_u = threadIdx.x % LPU, row_in_band = (threadIdx.x & 31) / LPU;
    int gw = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    int m = gw / wunits;
    int band = (gw - m * wunits) / nb, b = gw - m * wunits - band * nb;
    const int dm = SW / wunits, dband = (SW - dm * wunits) / nb, db = SW - dm * wunits - dband * nb;

    // issue the first loads before the table build so its latency is hidden
    float x[EPL];
    bool have = false;
    {
        const int r = band * GW + row_in_band, c = b * BS + lane_u * EPL;
        if (gw < total && r < n && c < n) { load_lane(Abase + (long long)m * strideA + (long long)r * n + c, x); have = true; }
    }
    build_tables<NC>(tab, code);
    const bool lean_launch = (NC == 16) && !tab.lut_bad && !tab.need_clamp && tab.perm_identity && !tab.tiny_thr;
    const unsigned *lut16 = tab.lut;
    const float lut_scale = tab.lut_scale;

    for (; gw < total; gw += SW) {
        const int r = band * GW + row_in_band, c = b * BS + lane_u * EPL;
        const bool unit_ok = r < n;
        const bool lane_ok = unit_ok && c < n;
        if (lane_ok) {
            if (!have) load_lane(Abase + (long long)m * strideA + (long long)r * n + c, x);
        } else {
#pragma unroll
            for (int j = 0; j < EPL; ++j) x[j] = 0.0f;
        }
        have = false;
        if (diag_base && lane_ok && (unsigned)(r - c) < (unsigned)EPL) {   // functional.py:574-578
#pragma unroll
            for (int j = 0; j < EPL; ++j)
                if (c + j == r) { diag_base[(long long)m * stride_diag + r] = x[j]; x[j] = 0.0f; }
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) amax = fmaxf(amax, fabsf(x[j]));
#pragma unroll
        for (int off = LPU / 2; off > 0; off >>= 1)
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        if (unit_ok && lane_u == 0) absmax_base[(long long)m * stride_absmax + (long long)r * nb + b] = amax;

        // Lean path (the hot one: 16-entry sorted codebook covering [-1, 1], no threshold within
        // 2^-50 of zero, every block scale of the warp in [2^-40, 2^60] or zero): q = x / absmax
        // through an exact reciprocal and two FMA corrections - bit-identical to the IEEE
        // division (functional.py:604) while nothing underflows; a |q| below 2^-60 only has to
        // keep its sign.  Anything else takes the out-of-line generic routine.
        const bool scale_ok = (amax >= 9.094947e-13f && amax <= 1.1529215e18f) || amax == 0.0f;
        const bool lean = lean_launch && __all_sync(0xffffffffu, scale_ok);
        if (lane_ok) {
            const long long e = (long long)r * n + c;         // flat element index, multiple of EPL
            unsigned char *out = out_base + (long long)m * stride_out;
            if constexpr (BITS == 4) {
                // codes are collected most-significant-nibble first (wq = wq << 4 | code), eight per
                // word, and the bytes of each word are reversed once at the end: element 2j ends up
                // in the high nibble of byte j (functional.py:733-734)
                constexpr int NW = EPL >= 8 ? EPL / 8 : 1;
                unsigned wq[NW];
#pragma unroll
                for (int i = 0; i < NW; ++i) wq[i] = 0;
                bool generic = !lean;
                if (lean) {
                    const float d = (amax == 0.0f) ? 1.0f : amax;
                    const float rcp = __frcp_rn(d);
                    unsigned nearest = 0xffffffffu;
#pragma unroll
                    for (int j = 0; j < EPL; ++j) {
                        // q0 = x * RN(1/d) is within 3 ulp of the IEEE quotient the reference forms
                        // (functional.py:604).  The cell word read as a float is the decision threshold to
                        // within 16 ulp (its low four bits hold the base index).  Unless q0 falls within
                        // 8 ulp of that 16-ulp bucket, q0 and the exact quotient lie on the same side of
                        // the threshold (and build_tables keeps thresholds 8 ulp away from cell
                        // borders, so a neighbouring cell gives the same answer): the code is exact.
                        const float q = x[j] * rcp;
                        const unsigned cellw = lut16[lut_cell_raw(q, lut_scale) & (kLutAlloc - 1)];
                        nearest = min(nearest, __float_as_uint(q) - (cellw & ~15u) + 8u);
                        const unsigned t = cellw + (q >= __uint_as_float(cellw) ? 1u : 0u);
                        wq[j / 8] = (wq[j / 8] << 4) | (t & 15u);
                    }
                    if (amax == 0.0f) {                       // functional.py:600-602
#pragma unroll
                        for (int i = 0; i < NW; ++i) wq[i] = 0;
                    }
                    generic = (nearest < 32u);                // rare: redo this lane with the exact division
                }
                if (generic) {
                    constexpr int PART = EPL > 8 ? 8 : EPL;
#pragma unroll
                    for (int h = 0; h < EPL / PART; ++h) {
                        LaneVals<PART> xv;
#pragma unroll
                        for (int j = 0; j < PART; ++j) xv.v[j] = x[h * PART + j];
                        const unsigned long long pk = quantize_lane_generic<NC, PART>(tab, xv, amax);
                        unsigned w = 0;
#pragma unroll
                        for (int j = 0; j < PART; ++j) w = (w << 4) | (unsigned)((pk >> (8 * j)) & 15u);
                        wq[h] = w;
                    }
                }
                if constexpr (EPL == 16) {
                    *reinterpret_cast<uint2 *>(out + (e >> 1)) = make_uint2(__byte_perm(wq[0], 0, 0x0123), __byte_perm(wq[1], 0, 0x0123));
                } else if constexpr (EPL == 8) {
                    *reinterpret_cast<unsigned *>(out + (e >> 1)) = __byte_perm(wq[0], 0, 0x0123);
                } else {
                    *reinterpret_cast<unsigned short *>(out + (e >> 1)) = (unsigned short)(((wq[0] >> 8) & 0xffu) | ((wq[0] & 0xffu) << 8));
                }
            } else {
                // 8-bit codes: always the out-of-line routine (binary search over 255 thresholds)
                int idx[EPL];
                constexpr int PART = EPL > 8 ? 8 : EPL;
#pragma unroll
                for (int h = 0; h < EPL / PART; ++h) {
                    LaneVals<PART> xv;
#pragma unroll
                    for (int j = 0; j < PART; ++j) xv.v[j] = x[h * PART + j];
                    const unsigned long long pk = quantize_lane_generic<NC, PART>(tab, xv, amax);
#pragma unroll
                    for (int j = 0; j < PART; ++j) idx[h * PART + j] = (int)((pk >> (8 * j)) & 255u);
                }
                unsigned w0 = 0, w1 = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) w0 |= (unsigned)idx[j] << (8 * j);
                if constexpr (EPL == 8) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) w1 |= (unsigned)idx[4 + j] << (8 * j);
                    *reinterpret_cast<uint2 *>(out + e) = make_uint2(w0, w1);
                } else {
                    *reinterpret_cast<unsigned *>(out + e) = w0;
                }
            }
        }
        b += db; band += dband; m += dm;
        if (b >= nb) { b -= nb; band += 1; }
        if (band >= bands) { band -= bands; m += 1; }
    }
}

// ------------------------------------------------------------------------------------
// Quantize, generic path: any order, any alignment, any supported block size.
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
k_absmax_generic(const T *__restrict__ Abase, long long strideA, int n, int nb, int bs,
                 float *__restrict__ absmax_base, long long stride_absmax,
                 float *__restrict__ diag_base, long long stride_diag) {
    const int m = blockIdx.y;
    const T *A = Abase + (long long)m * strideA;
    float *absmax = absmax_base + (long long)m * stride_absmax;
    float *diag = diag_base ? diag_base + (long long)m * stride_diag : nullptr;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * kThreads) >> 5;
    const int units = n * nb;
    for (int u = (blockIdx.x * kThreads + threadIdx.x) >> 5; u < units; u += warps) {
        const int r = u / nb, b = u - r * nb;
        const int c0 = b * bs, c1 = min(c0 + bs, n);
        float amax = 0.0f;
        for (int c = c0 + lane; c < c1; c += 32) {
            float x = to_f32<T>(A[(long long)r * n + c]);
            if (diag && c == r) { diag[r] = x; x = 0.0f; }
            amax = fmaxf(amax, fabsf(x));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        if (lane == 0) absmax[u] = amax;
    }
}

template <typename T, int BITS>
__global__ void __launch_bounds__(kThreads)
k_encode_generic(const T *__restrict__ Abase, long long strideA, const float *__restrict__ code,
                 int n, int nb, int bs, const float *__restrict__ absmax_base, long long stride_absmax,
                 int diagreal, unsigned char *__restrict__ out_base, long long stride_out) {
    constexpr int NC = 1 << BITS;
    constexpr int PER = 8 / BITS;                            // elements per output byte
    __shared__ CodeTables<NC> tab;
    build_tables<NC>(tab, code);
    const int m = blockIdx.y;
    const T *A = Abase + (long long)m * strideA;
    const float *absmax = absmax_base + (long long)m * stride_absmax;
    unsigned char *out = out_base + (long long)m * stride_out;
    const long long total = (long long)n * n;
    const long long nbytes = (total + PER - 1) / PER;
    for (long long byte = (long long)blockIdx.x * kThreads + threadIdx.x; byte < nbytes;
         byte += (long long)gridDim.x * kThreads) {
        unsigned v = 0;
#pragma unroll
        for (int h = 0; h < PER; ++h) {
            const long long e = byte * PER + h;
            int k = 0;                                        // padding nibble is 0 (functional.py:724-732)
            if (e < total) {
                const int r = (int)(e / n), c = (int)(e - (long long)r * n);
                float x = to_f32<T>(A[e]);
                if (diagreal && r == c) x = 0.0f;
                const float amax = absmax[(long long)r * nb + c / bs];
                if (amax != 0.0f) {
                    float q = __fdiv_rn(x, amax);
                    if (tab.need_clamp) q = fminf(fmaxf(q, tab.cmin), tab.cmax);
                    k = tab.perm[code_index_search<NC>(tab, q)];
                }
            }
            v = (BITS == 4) ? ((v << 4) | (unsigned)k) : (unsigned)k;
        }
        out[byte] = (unsigned char)v;
    }
}

// ------------------------------------------------------------------------------------
// Dequantize.
// ------------------------------------------------------------------------------------
template <typename T, int EPL> __device__ __forceinline__ void store_vec(T *p, const float (&v)[EPL]);
template <> __device__ __forceinline__ void store_vec<float, 4>(float *p, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store_vec<float, 8>(float *p, const float (&v)[8]) {
    stg256(p, v);                                             // launcher guarantees 32-byte alignment
}
__device__ __forceinline__ unsigned pack_bf16x2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);           // .x = a (low half), .y = b
    return *reinterpret_cast<unsigned *>(&h);
}
template <> __device__ __forceinline__ void store_vec<__nv_bfloat16, 4>(__nv_bfloat16 *p, const float (&v)[4]) {
    *reinterpret_cast<uint2 *>(p) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
}
template <> __device__ __forceinline__ void store_vec<__nv_bfloat16, 8>(__nv_bfloat16 *p, const float (&v)[8]) {
    *reinterpret_cast<uint4 *>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                               pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}

// Vector path: n % EPL == 0, aligned buffers; any supported block size (power of two).
template <typename T, int BITS, int EPL>
__global__ void __launch_bounds__(kThreads)
k_dequantize_vec(const unsigned char *__restrict__ in_base, long long stride_in, const float *__restrict__ code,
                 int n, int nb, int bs_shift, const float *__restrict__ absmax_base, long long stride_absmax,
                 const float *__restrict__ diag_base, long long stride_diag,
                 T *__restrict__ out_base, long long stride_out) {
    constexpr int NC = 1 << BITS;
    __shared__ float2 pair_lut[BITS == 4 ? 256 : 1];          // byte -> (high-nibble value, low-nibble value)
    __shared__ float code_s[BITS == 8 ? 256 : 16];
    for (int i = threadIdx.x; i < NC; i += blockDim.x) code_s[i] = code[i];
    __syncthreads();
    if (BITS == 4)
        for (int i = threadIdx.x; i < 256; i += blockDim.x) pair_lut[i] = make_float2(code_s[i >> 4], code_s[i & 15]);
    __syncthreads();

    const int m = blockIdx.y;
    const unsigned char *in = in_base + (long long)m * stride_in;
    const float *absmax = absmax_base + (long long)m * stride_absmax;
    const float *diag = diag_base ? diag_base + (long long)m * stride_diag : nullptr;
    T *out = out_base + (long long)m * stride_out;

    const int chunks_per_row = n / EPL;
    const int chunks = n * chunks_per_row;
    const int S = gridDim.x * kThreads;
    int t = blockIdx.x * kThreads + threadIdx.x;
    int r = t / chunks_per_row, cc = t - r * chunks_per_row;
    const int dr = S / chunks_per_row, dc = S - dr * chunks_per_row;
#pragma unroll 4
    for (; t < chunks; t += S) {
        const int c = cc * EPL;
        const long long e = (long long)r * n + c;
        const float amax = __ldg(absmax + (long long)r * nb + (c >> bs_shift));
        const float z = (amax == 0.0f) ? 0.0f : -0.0f;        // exact +0.0 for all-zero blocks (functional.py:663-665)
        float v[EPL];
        if constexpr (BITS == 4) {
            unsigned w;
            if constexpr (EPL == 8) w = __ldg(reinterpret_cast<const unsigned *>(in + (e >> 1)));
            else w = __ldg(reinterpret_cast<const unsigned short *>(in + (e >> 1)));
#pragma unroll
            for (int j = 0; j < EPL / 2; ++j) {
                float2 p = pair_lut[(w >> (8 * j)) & 255u];
                v[2 * j] = fmaf(p.x, amax, z);
                v[2 * j + 1] = fmaf(p.y, amax, z);
            }
        } else {
            unsigned w0, w1 = 0;
            if constexpr (EPL == 8) {
                uint2 ww = __ldg(reinterpret_cast<const uint2 *>(in + e));
                w0 = ww.x; w1 = ww.y;
            } else {
                w0 = __ldg(reinterpret_cast<const unsigned *>(in + e));
            }
#pragma unroll
            for (int j = 0; j < EPL; ++j) {
                unsigned byte = ((j < 4 ? w0 : w1) >> (8 * (j & 3))) & 255u;
                v[j] = fmaf(code_s[byte], amax, z);
            }
        }
        if (diag && r >= c && r < c + EPL) {                  // functional.py:673-678
            const float d = diag[r];
#pragma unroll
            for (int j = 0; j < EPL; ++j)
                if (c + j == r) v[j] = d;
        }
        store_vec<T, EPL>(out + e, v);
        r += dr; cc += dc;
        if (cc >= chunks_per_row) { cc -= chunks_per_row; r += 1; }
    }
}

// ------------------------------------------------------------------------------------
// Dequantize straight into the operand format of the tcgen05 products: two bf16 planes
// (hi = bf16(x), lo = bf16(x - hi)) with row pitch ldp.  Output matrix j is taken from state
// slot slots[j] (or j when slots == nullptr), so a product's batch can be assembled from
// scattered slots of an arena without an fp32 copy, a stack and a split pass in between.
// EPL = 8 elements per thread (one 32/64-bit code load, one 128-bit store per plane) or, with
// 32-byte aligned rows, 16 (one 256-bit store per plane).
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void stg256u(void *p, const unsigned (&v)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

// Largest magnitude a dequantized state matrix can hold: max over its block scales and its fp32
// diagonal (|code| <= 1).  One CTA per output matrix; amax[m] belongs to state slot slots[m].
__global__ void __launch_bounds__(256)
k_state_amax(const float *__restrict__ absmax_base, long long stride_absmax, int n_absmax,
             const float *__restrict__ diag_base, long long stride_diag, int n_diag,
             const int *__restrict__ slots, float *__restrict__ amax, int *__restrict__ exp_out = nullptr, int target = 0) {
    const int m = blockIdx.x;
    const long long src = slots ? (long long)slots[m] : (long long)m;
    // four independent loads in flight per thread: a matrix has 9 K - 23 K block scales and this CTA is
    // alone with them, so the loop is bound by load latency, not bandwidth
    float v0 = 0.0f, v1 = 0.0f, v2 = 0.0f, v3 = 0.0f;
    const float *am = absmax_base + src * stride_absmax;
    const int step = blockDim.x;
    int i = threadIdx.x;
    for (; i + 3 * step < n_absmax; i += 4 * step) {
        const float a = __ldg(am + i), b = __ldg(am + i + step), c = __ldg(am + i + 2 * step), d = __ldg(am + i + 3 * step);
        v0 = fmaxf(v0, fabsf(a)); v1 = fmaxf(v1, fabsf(b)); v2 = fmaxf(v2, fabsf(c)); v3 = fmaxf(v3, fabsf(d));
    }
    for (; i < n_absmax; i += step) v0 = fmaxf(v0, fabsf(__ldg(am + i)));
    float v = fmaxf(fmaxf(v0, v1), fmaxf(v2, v3));
    if (diag_base)
        for (int k = threadIdx.x; k < n_diag; k += blockDim.x) v = fmaxf(v, fabsf(__ldg(diag_base + src * stride_diag + k)));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    __shared__ float red[8];
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) v = fmaxf(v, red[i]);
        if (amax) amax[m] = v;
        if (exp_out) exp_out[m] = exponent_for(v, target);
    }
}

// F16: the planes are scaled fp16 planes (entry = value * 2^e, e from amax[m] and `target`,
// written to exp_out[m]); otherwise plain bf16 planes.
template <int BITS, int EPL, bool F16>
__global__ void __launch_bounds__(kThreads)
k_dequantize_planes(const unsigned char *__restrict__ in_base, long long stride_in, const float *__restrict__ code,
                    int n, int nb, int bs_shift, const float *__restrict__ absmax_base, long long stride_absmax,
                    const float *__restrict__ diag_base, long long stride_diag, const int *__restrict__ slots,
                    __nv_bfloat16 *__restrict__ hi_base, __nv_bfloat16 *__restrict__ lo_base, long long ldp, long long strideP,
                    const float *__restrict__ amax, int target, int *__restrict__ exp_out) {
    constexpr int NC = 1 << BITS;
    __shared__ float2 pair_lut[BITS == 4 ? 256 : 1];
    __shared__ float code_s[BITS == 8 ? 256 : 16];
    for (int i = threadIdx.x; i < NC; i += blockDim.x) code_s[i] = code[i];
    __syncthreads();
    if (BITS == 4)
        for (int i = threadIdx.x; i < 256; i += blockDim.x) pair_lut[i] = make_float2(code_s[i >> 4], code_s[i & 15]);
    __syncthreads();

    const int m = blockIdx.y;
    const long long src = slots ? (long long)slots[m] : (long long)m;
    const unsigned char *in = in_base + src * stride_in;
    const float *absmax = absmax_base + src * stride_absmax;
    const float *diag = diag_base ? diag_base + src * stride_diag : nullptr;
    __nv_bfloat16 *hi = hi_base + (long long)m * strideP, *lo = lo_base + (long long)m * strideP;
    float two_e = 1.0f;
    if constexpr (F16) {
        const int e = exponent_for(amax[m], target);
        two_e = exp2f((float)e);
        if (exp_out && blockIdx.x == 0 && threadIdx.x == 0) exp_out[m] = e;
    }

    const int chunks_per_row = n / EPL;
    const int chunks = n * chunks_per_row;
    const int S = gridDim.x * kThreads;
    int t = blockIdx.x * kThreads + threadIdx.x;
    int r = t / chunks_per_row, cc = t - r * chunks_per_row;
    const int dr = S / chunks_per_row, dc = S - dr * chunks_per_row;
#pragma unroll 2
    for (; t < chunks; t += S) {
        const int c = cc * EPL;
        const long long e = (long long)r * n + c;
        const float amax = __ldg(absmax + (long long)r * nb + (c >> bs_shift));
        const float z = (amax == 0.0f) ? 0.0f : -0.0f;        // exact +0.0 for all-zero blocks
        float v[EPL];
        if constexpr (BITS == 4) {
            unsigned w[EPL / 8];
            if constexpr (EPL == 16) {
                const uint2 ww = __ldg(reinterpret_cast<const uint2 *>(in + (e >> 1)));
                w[0] = ww.x; w[1] = ww.y;
            } else {
                w[0] = __ldg(reinterpret_cast<const unsigned *>(in + (e >> 1)));
            }
#pragma unroll
            for (int j = 0; j < EPL / 2; ++j) {
                const float2 pr = pair_lut[(w[j / 4] >> (8 * (j & 3))) & 255u];
                v[2 * j] = fmaf(pr.x, amax, z);
                v[2 * j + 1] = fmaf(pr.y, amax, z);
            }
        } else {
            unsigned w[EPL / 4];
            if constexpr (EPL == 16) {
                const uint4 ww = __ldg(reinterpret_cast<const uint4 *>(in + e));
                w[0] = ww.x; w[1] = ww.y; w[2] = ww.z; w[3] = ww.w;
            } else {
                const uint2 ww = __ldg(reinterpret_cast<const uint2 *>(in + e));
                w[0] = ww.x; w[1] = ww.y;
            }
#pragma unroll
            for (int j = 0; j < EPL; ++j) v[j] = fmaf(code_s[(w[j / 4] >> (8 * (j & 3))) & 255u], amax, z);
        }
        if (diag && (unsigned)(r - c) < (unsigned)EPL) {
            const float d = diag[r];
#pragma unroll
            for (int j = 0; j < EPL; ++j)
                if (c + j == r) v[j] = d;
        }
        unsigned h[EPL / 2], l[EPL / 2];
#pragma unroll
        for (int j = 0; j < EPL / 2; ++j) {
            if constexpr (F16) {
                const float a0 = v[2 * j] * two_e, a1 = v[2 * j + 1] * two_e;
                const __half h0 = __float2half_rn(a0), h1 = __float2half_rn(a1);
                const __half l0 = __float2half_rn(a0 - __half2float(h0)), l1 = __float2half_rn(a1 - __half2float(h1));
                h[j] = (unsigned)__half_as_ushort(h0) | ((unsigned)__half_as_ushort(h1) << 16);
                l[j] = (unsigned)__half_as_ushort(l0) | ((unsigned)__half_as_ushort(l1) << 16);
            } else {
                const __nv_bfloat16 h0 = __float2bfloat16_rn(v[2 * j]), h1 = __float2bfloat16_rn(v[2 * j + 1]);
                const __nv_bfloat16 l0 = __float2bfloat16_rn(v[2 * j] - __bfloat162float(h0));
                const __nv_bfloat16 l1 = __float2bfloat16_rn(v[2 * j + 1] - __bfloat162float(h1));
                h[j] = (unsigned)__bfloat16_as_ushort(h0) | ((unsigned)__bfloat16_as_ushort(h1) << 16);
                l[j] = (unsigned)__bfloat16_as_ushort(l0) | ((unsigned)__bfloat16_as_ushort(l1) << 16);
            }
        }
        const long long o = (long long)r * ldp + c;
        if constexpr (EPL == 16) {
            stg256u(hi + o, h);
            stg256u(lo + o, l);
        } else {
            *reinterpret_cast<uint4 *>(hi + o) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4 *>(lo + o) = make_uint4(l[0], l[1], l[2], l[3]);
        }
        r += dr; cc += dc;
        if (cc >= chunks_per_row) { cc -= chunks_per_row; r += 1; }
    }
}

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T, int BITS>
__global__ void __launch_bounds__(kThreads)
k_dequantize_generic(const unsigned char *__restrict__ in_base, long long stride_in, const float *__restrict__ code,
                     int n, int nb, int bs, const float *__restrict__ absmax_base, long long stride_absmax,
                     const float *__restrict__ diag_base, long long stride_diag,
                     T *__restrict__ out_base, long long stride_out) {
    constexpr int NC = 1 << BITS;
    __shared__ float code_s[NC];
    for (int i = threadIdx.x; i < NC; i += blockDim.x) code_s[i] = code[i];
    __syncthreads();
    const int m = blockIdx.y;
    const unsigned char *in = in_base + (long long)m * stride_in;
    const float *absmax = absmax_base + (long long)m * stride_absmax;
    const float *diag = diag_base ? diag_base + (long long)m * stride_diag : nullptr;
    T *out = out_base + (long long)m * stride_out;
    const long long total = (long long)n * n;
    for (long long e = (long long)blockIdx.x * kThreads + threadIdx.x; e < total; e += (long long)gridDim.x * kThreads) {
        const int r = (int)(e / n), c = (int)(e - (long long)r * n);
        int k;
        if (BITS == 8) k = in[e];
        else { unsigned char byte = in[e >> 1]; k = (e & 1) ? (byte & 15) : (byte >> 4); }
        const float amax = absmax[(long long)r * nb + c / bs];
        float v = fmaf(code_s[k], amax, (amax == 0.0f) ? 0.0f : -0.0f);
        if (diag && r == c) v = diag[r];
        out[e] = from_f32<T>(v);
    }
}

// ------------------------------------------------------------------------------------
// Self-test of the fast division: counts pairs (x, d), d in [2^-40, 2^60], |x| <= d, whose
// reciprocal-based quotient differs in any bit from the IEEE division (quotients below 2^-60
// in magnitude are exempt, as in the quantizer).  Pairs come from a counter-based hash.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned mix32(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull; z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return (unsigned)((z ^ (z >> 31)) >> 16);
}
__global__ void k_selftest_division(unsigned long long seed, unsigned long long pairs, unsigned long long *mismatches) {
    unsigned long long bad = 0;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < pairs;
         i += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned a = mix32(seed + 2 * i), b = mix32(seed + 2 * i + 1);
        // d: exponent in [-40, 60), random mantissa; x = d * (fraction in [-1, 1]) with a random small exponent drop
        const int ed = (int)(a % 100u) - 40 + 127;
        const float d = __uint_as_float(((unsigned)ed << 23) | (b & 0x7FFFFFu));
        const unsigned c = mix32(seed ^ (i * 0xD1342543DE82EF95ull));
        const int drop = (c >> 24) % 40;                       // |x| spans 40 binades below d
        float x = __uint_as_float(((unsigned)(ed - drop) << 23) | (c & 0x7FFFFFu));
        if (fabsf(x) > d) x = d;
        if (a & 0x80000000u) x = -x;
        if ((c & 0xFF00u) == 0) x = (c & 1) ? d : -d;           // exact +-1 quotients
        const float q_ref = __fdiv_rn(x, d);
        const float q = div_by_recip(x, d, __frcp_rn(d));
        if (fabsf(q_ref) >= 8.6736174e-19f && __float_as_uint(q) != __float_as_uint(q_ref)) ++bad;   // 2^-60
    }
    if (bad) atomicAdd(mismatches, bad);
}

int launch_selftest_division(unsigned long long seed, unsigned long long pairs, unsigned long long *mismatches_dev,
                             cudaStream_t s) {
    if (!mismatches_dev) return record(QT_ERR_ARG);
    k_selftest_division<<<148 * 8, 256, 0, s>>>(seed, pairs, mismatches_dev);
    count_launch(1);
    return check_launch();
}

// ------------------------------------------------------------------------------------
// Host launchers.
// ------------------------------------------------------------------------------------
static int sm_count() { return device_sm_count(); }

static inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// grid.x for `work_items` thread-iterations of one matrix, `count` matrices in grid.y:
// enough CTAs to fill the machine a few times over, at least `min_iters` iterations per
// thread where the matrix is large enough to amortise the per-CTA table build.
static unsigned grid_x_for(long long thread_iters, int count, int min_iters) {
    long long ctas = (thread_iters + (long long)kThreads * min_iters - 1) / ((long long)kThreads * min_iters);
    const long long target = (long long)sm_count() * 8;      // resident CTAs of 256 threads per SM
    long long per_matrix_cap = (target * 4 + count - 1) / count;
    if (per_matrix_cap < 1) per_matrix_cap = 1;
    if (ctas > per_matrix_cap) ctas = per_matrix_cap;
    if (ctas < 1) ctas = 1;
    return (unsigned)ctas;
}

template <typename T, int BITS>
static void launch_quantize_typed(const QuantArgs &a, cudaStream_t s) {
    const int n = a.n, nb = (n + a.bs - 1) / a.bs;
    const T *A = static_cast<const T *>(a.A);
    const size_t esz = sizeof(T);
    const bool strides_ok8 = (a.strideA * (long long)esz) % 16 == 0 && a.stride_out % 4 == 0;
    const bool strides_ok4 = (a.strideA * (long long)esz) % (4 * esz) == 0 && a.stride_out % (BITS == 4 ? 2 : 4) == 0;
    const bool ptr_ok8 = aligned(A, 16) && aligned(a.out, BITS == 4 ? 4 : 8);
    const bool ptr_ok4 = aligned(A, 4 * esz) && aligned(a.out, BITS == 4 ? 2 : 4);
    const bool many = a.count > 1;
    int epl = 0;
    if (a.bs <= 256) {
        if (n % 8 == 0 && ptr_ok8 && (!many || strides_ok8)) epl = 8;
        else if (n % 4 == 0 && ptr_ok4 && (!many || strides_ok4) && a.bs <= 128) epl = 4;
    }
    // 4-bit, block 64 (the optimizers' configuration): 16 elements per lane, 4 lanes per block
    if (BITS == 4 && a.bs == 64 && epl == 8 && n % 16 == 0 && aligned(a.out, 8) && (!many || a.stride_out % 8 == 0) &&
        (!many || (a.strideA * (long long)esz) % 16 == 0))
        epl = 16;
    if (epl) {
        const int lpu = a.bs / epl;
        // every CTA builds the code tables once: exactly one resident wave (or fewer CTAs when the
        // batch is small), striding over the units of the whole batch
        const long long wunits = (long long)((n + 32 / lpu - 1) / (32 / lpu)) * nb;   // warp units per matrix
        if (wunits * a.count >= (1ll << 31) - (1ll << 24) && a.count > 1) {   // warp-unit numbers are 32-bit in the kernel
            const int half = a.count / 2;
            QuantArgs lo = a, hi = a;
            lo.count = half;
            hi.count = a.count - half;
            hi.A = (const char *)a.A + (long long)half * a.strideA * (long long)esz;
            hi.absmax = a.absmax + (long long)half * a.stride_absmax;
            hi.diag = a.diag ? a.diag + (long long)half * a.stride_diag : nullptr;
            hi.out = a.out + (long long)half * a.stride_out;
            launch_quantize_typed<T, BITS>(lo, s);
            launch_quantize_typed<T, BITS>(hi, s);
            return;
        }
        const int resident = 4;                              // the kernels' launch bounds
        // 256-bit loads need every lane's 16 elements on a 32-byte boundary
        const int wide = (epl == 16 && aligned(A, 32) && ((long long)n * (long long)esz) % 32 == 0 &&
                          (!many || (a.strideA * (long long)esz) % 32 == 0)) ? 1 : 0;
        long long ctas = (long long)sm_count() * resident;
        const long long needed = (wunits * a.count + kThreads / 32 - 1) / (kThreads / 32);
        if (ctas > needed) ctas = needed;
        if (ctas < 1) ctas = 1;
        dim3 grid((unsigned)ctas);
#define QT_LAUNCH_Q(E, L)                                                                          \
        k_quantize_vec<T, BITS, E, L><<<grid, kThreads, 0, s>>>(A, a.strideA, a.code, n, nb, a.count, a.absmax, \
            a.stride_absmax, a.diag, a.stride_diag, a.out, a.stride_out, wide)
        if constexpr (BITS == 4) { if (epl == 16) { QT_LAUNCH_Q(16, 4); count_launch(1); return; } }
        if (epl == 8 && lpu == 8) QT_LAUNCH_Q(8, 8);
        else if (epl == 8 && lpu == 16) QT_LAUNCH_Q(8, 16);
        else if (epl == 8 && lpu == 32) QT_LAUNCH_Q(8, 32);
        else if (epl == 4 && lpu == 16) QT_LAUNCH_Q(4, 16);
        else QT_LAUNCH_Q(4, 32);
#undef QT_LAUNCH_Q
        count_launch(1);
        return;
    }
    const long long units = (long long)n * nb;
    dim3 g1(grid_x_for(units * 32, a.count, 1), a.count);
    k_absmax_generic<T><<<g1, kThreads, 0, s>>>(A, a.strideA, n, nb, a.bs, a.absmax, a.stride_absmax, a.diag, a.stride_diag);
    const long long nbytes = ((long long)n * n * BITS + 7) / 8;
    dim3 g2(grid_x_for(nbytes, a.count, 4), a.count);
    k_encode_generic<T, BITS><<<g2, kThreads, 0, s>>>(A, a.strideA, a.code, n, nb, a.bs, a.absmax, a.stride_absmax,
                                                     a.diag != nullptr, a.out, a.stride_out);
    count_launch(2);
}

int launch_quantize(const QuantArgs &a, cudaStream_t s) {
    if (a.bits != 4 && a.bits != 8) return record(QT_ERR_BITS);
    if (!valid_blocksize(a.bs)) return record(QT_ERR_BLOCKSIZE);
    if (a.a_dtype != QT_F32 && a.a_dtype != QT_BF16) return record(QT_ERR_DTYPE);
    if (a.n < 0 || a.count < 0 || a.n > 46340 || a.count > 65535) return record(QT_ERR_ARG);
    if (a.n == 0 || a.count == 0) return record(QT_OK);
    if (!a.A || !a.code || !a.absmax || !a.out) return record(QT_ERR_ARG);
    if (!aligned(a.absmax, 4) || !aligned(a.code, 4) || (a.diag && !aligned(a.diag, 4))) return record(QT_ERR_ARG);
    if (!aligned(a.A, a.a_dtype == QT_F32 ? 4 : 2)) return record(QT_ERR_ARG);
    if (a.a_dtype == QT_F32) {
        if (a.bits == 4) launch_quantize_typed<float, 4>(a, s); else launch_quantize_typed<float, 8>(a, s);
    } else {
        if (a.bits == 4) launch_quantize_typed<__nv_bfloat16, 4>(a, s); else launch_quantize_typed<__nv_bfloat16, 8>(a, s);
    }
    return check_launch();
}

template <typename T, int BITS>
static void launch_dequantize_typed(const DequantArgs &a, cudaStream_t s) {
    const int n = a.n, nb = (n + a.bs - 1) / a.bs;
    T *out = static_cast<T *>(a.out);
    const size_t esz = sizeof(T);
    int bs_shift = 0;
    while ((1 << bs_shift) < a.bs) ++bs_shift;
    const bool many = a.count > 1;
    auto ok = [&](int epl) {
        // fp32 x 8 is one 256-bit store (32-byte aligned); everything else is at most 128 bits
        const size_t in_bytes = (size_t)epl * BITS / 8, out_bytes = (size_t)(epl * esz > 16 ? (esz == 4 ? 32 : 16) : epl * esz);
        if (n % epl) return false;
        if (!aligned(a.A, in_bytes) || !aligned(out, out_bytes)) return false;
        if (many && (a.strideA % (long long)in_bytes || (a.stride_out * (long long)esz) % (long long)out_bytes)) return false;
        return true;
    };
    // 8 elements per thread make one store: 256 bits of fp32 or 128 bits of bf16; otherwise 4
    // elements (one 128-bit fp32 store).
    int epl = ok(8) ? 8 : (ok(4) ? 4 : 0);
    if (epl) {
        const long long chunks = (long long)n * (n / epl);
        dim3 grid(grid_x_for(chunks, a.count, 4), a.count);
        if (epl == 8)
            k_dequantize_vec<T, BITS, 8><<<grid, kThreads, 0, s>>>(a.A, a.strideA, a.code, n, nb, bs_shift, a.absmax,
                a.stride_absmax, a.diag, a.stride_diag, out, a.stride_out);
        else
            k_dequantize_vec<T, BITS, 4><<<grid, kThreads, 0, s>>>(a.A, a.strideA, a.code, n, nb, bs_shift, a.absmax,
                a.stride_absmax, a.diag, a.stride_diag, out, a.stride_out);
        count_launch(1);
        return;
    }
    count_launch(1);
    dim3 grid(grid_x_for((long long)n * n, a.count, 4), a.count);
    k_dequantize_generic<T, BITS><<<grid, kThreads, 0, s>>>(a.A, a.strideA, a.code, n, nb, a.bs, a.absmax, a.stride_absmax,
                                                           a.diag, a.stride_diag, out, a.stride_out);
}

int launch_dequantize(const DequantArgs &a, cudaStream_t s) {
    if (a.bits != 4 && a.bits != 8) return record(QT_ERR_BITS);
    if (!valid_blocksize(a.bs)) return record(QT_ERR_BLOCKSIZE);
    if (a.out_dtype != QT_F32 && a.out_dtype != QT_BF16) return record(QT_ERR_DTYPE);
    if (a.n < 0 || a.count < 0 || a.n > 46340 || a.count > 65535) return record(QT_ERR_ARG);
    if (a.n == 0 || a.count == 0) return record(QT_OK);
    if (!a.A || !a.code || !a.absmax || !a.out) return record(QT_ERR_ARG);
    if (!aligned(a.absmax, 4) || !aligned(a.code, 4) || (a.diag && !aligned(a.diag, 4))) return record(QT_ERR_ARG);
    if (!aligned(a.out, a.out_dtype == QT_F32 ? 4 : 2)) return record(QT_ERR_ARG);
    if (a.out_dtype == QT_F32) {
        if (a.bits == 4) launch_dequantize_typed<float, 4>(a, s); else launch_dequantize_typed<float, 8>(a, s);
    } else {
        if (a.bits == 4) launch_dequantize_typed<__nv_bfloat16, 4>(a, s); else launch_dequantize_typed<__nv_bfloat16, 8>(a, s);
    }
    return check_launch();
}

int launch_state_exponents(const float *absmax, long long stride_absmax, int n_absmax, const float *diag, long long stride_diag,
                           int n_diag, const int *slots, int count, int target, int *exp_out, cudaStream_t s) {
    if (count < 0 || n_absmax < 0 || !absmax || !exp_out) return record(QT_ERR_ARG);
    if (count == 0) return record(QT_OK);
    k_state_amax<<<count, 256, 0, s>>>(absmax, stride_absmax, n_absmax, diag, stride_diag, n_diag, slots, nullptr, exp_out, target);
    count_launch(1);
    return check_launch();
}

int launch_dequantize_planes(const DequantArgs &a, const int *slots, void *hi, void *lo, long long ldp, long long strideP,
                             cudaStream_t s, float *amax_scratch, int target, int *exp_out) {
    if (a.bits != 4 && a.bits != 8) return record(QT_ERR_BITS);
    if (!valid_blocksize(a.bs)) return record(QT_ERR_BLOCKSIZE);
    if (a.n < 0 || a.count < 0 || a.n > 46340 || a.count > 65535) return record(QT_ERR_ARG);
    if (a.n == 0 || a.count == 0) return record(QT_OK);
    if (!a.A || !a.code || !a.absmax || !hi || !lo) return record(QT_ERR_ARG);
    // eight elements per thread: 16-byte plane stores, 4/8-byte code loads
    if (a.n % 8 || ldp % 8 || strideP % 8 || !aligned(hi, 16) || !aligned(lo, 16) || ldp < a.n) return record(QT_ERR_UNSUPPORTED);
    const int in_bytes = a.bits == 4 ? 4 : 8;
    if (!aligned(a.A, in_bytes) || a.strideA % in_bytes) return record(QT_ERR_UNSUPPORTED);
    if (!aligned(a.absmax, 4) || !aligned(a.code, 4) || (a.diag && !aligned(a.diag, 4))) return record(QT_ERR_ARG);
    const int n = a.n, nb = (n + a.bs - 1) / a.bs;
    int bs_shift = 0;
    while ((1 << bs_shift) < a.bs) ++bs_shift;
    // 16 elements per thread: 256-bit plane stores (32-byte rows) and 8/16-byte code loads
    const int in16 = a.bits == 4 ? 8 : 16;
    const bool wide = n % 16 == 0 && ldp % 16 == 0 && strideP % 16 == 0 && aligned(hi, 32) && aligned(lo, 32) &&
                      aligned(a.A, in16) && a.strideA % in16 == 0 && a.bs >= 16;
    dim3 grid(grid_x_for((long long)n * (n / (wide ? 16 : 8)), a.count, 4), a.count);
    const bool f16 = amax_scratch != nullptr;
    if (f16) {
        k_state_amax<<<a.count, 256, 0, s>>>(a.absmax, a.stride_absmax, n * nb, a.diag, a.stride_diag, n, slots, amax_scratch);
        count_launch(1);
    }
#define QT_DQP(B, E, H)                                                                                                 \
    k_dequantize_planes<B, E, H><<<grid, kThreads, 0, s>>>(a.A, a.strideA, a.code, n, nb, bs_shift, a.absmax, a.stride_absmax, \
        a.diag, a.stride_diag, slots, static_cast<__nv_bfloat16 *>(hi), static_cast<__nv_bfloat16 *>(lo), ldp, strideP,   \
        amax_scratch, target, exp_out)
    if (f16) {
        if (a.bits == 4) { if (wide) QT_DQP(4, 16, true); else QT_DQP(4, 8, true); }
        else { if (wide) QT_DQP(8, 16, true); else QT_DQP(8, 8, true); }
    } else {
        if (a.bits == 4) { if (wide) QT_DQP(4, 16, false); else QT_DQP(4, 8, false); }
        else { if (wide) QT_DQP(8, 16, false); else QT_DQP(8, 8, false); }
    }
#undef QT_DQP
    count_launch(1);
    return check_launch();
}

}  // namespace qt
