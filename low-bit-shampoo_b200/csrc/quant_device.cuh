// Device-side pieces of the blockwise quantizer that more than one kernel needs: the per-CTA
// codebook tables (exact decision thresholds + packed lookup table), the exact division and the
// generic per-lane routine.  Included by the stand-alone quantize kernels and by the GEMM whose
// epilogue writes 4-bit state.
#pragma once
#include "qt_common.cuh"
#include <math_constants.h>

namespace qt {

static constexpr int kLutAlloc = 2048;        // cells allocated; the finest grid uses 2*512+1 of them
static constexpr float kLutCoarseScale = 127.0f;   // coarse grid: cells 0..254, so an 8-bit mask is a safe index

// ------------------------------------------------------------------------------------
// Codebook tables, built per CTA in shared memory.
// ------------------------------------------------------------------------------------
static constexpr int kCells8 = 2048;                         // cells over [-1, 1] for 256-entry codebooks
template <int NC>
struct CodeTables {
    float raw[NC];
    float sorted[NC];
    float thr[NC];            // thr[j], j < NC-1: smallest q that rounds up from sorted[j]; thr[NC-1] = +inf
    unsigned char perm[NC];   // sorted position -> caller's code index
    float cmin, cmax;
    int perm_identity;
    int need_clamp;
    int lut_bad;
    int tiny_thr;             // some decision threshold has |t| < 2^-50: quotients must be exact even when tiny
    int thr_cell[NC];         // lookup-table cell of each threshold
    float lut_scale;          // cells per unit of q: 127 (255 cells) when that separates the thresholds, else 512
    // One 32-bit word per cell of q in [-1, 1]: bits 31..4 = the threshold inside the cell (or +inf)
    // with its low four mantissa bits cleared, bits 3..0 = number of thresholds in lower cells.
    // A 4-byte cell halves the shared-memory wavefronts of a warp's 32 scattered lookups compared
    // with {float threshold, int base}; the 16-ulp bucket around the threshold that the cleared bits
    // cannot resolve is decided against the exact threshold (rare).
    unsigned lut[NC == 16 ? kLutAlloc : 1];
    // 256-entry codebooks: 2049 cells over [-1, 1]; per cell the number of thresholds in lower cells
    // (low byte) and in the cell itself (high byte).  A quotient is compared against the exact
    // thresholds of its own cell only (one on average) instead of eight steps of a binary search.
    unsigned short cell8[NC == 256 ? kCells8 + 1 : 1];
};

// Cell of a quotient on the 256-entry grid: floor(1024 q + 1024) clamped to [0, 2048].  Monotone in q.
__device__ __forceinline__ int cell8_of(float q) {
    return __float2int_rd(fminf(fmaxf(fmaf(q, 1024.0f, 1024.0f), 0.0f), (float)kCells8));
}

__device__ __forceinline__ long long float_key(float f) {
    int i = __float_as_int(f);
    return (long long)(i >= 0 ? i : (i ^ 0x7fffffff));
}
__device__ __forceinline__ float key_float(long long k) {
    int i = (int)k;
    return __int_as_float(i >= 0 ? i : (i ^ 0x7fffffff));
}
// Cell of q in [-1, 1] on a grid of `scale` cells per unit: round(q*scale + scale), taken from the
// mantissa of the sum with 2^23 (no float-to-int conversion).  Monotone in q, which is all the table
// needs.  The caller masks the result with kLutAlloc-1, which also removes the exponent bits.
__device__ __forceinline__ int lut_cell_raw(float v, float scale) {
    return __float_as_int(fmaf(v, scale, scale + 8388608.0f));
}

template <int NC>
__device__ void build_tables(CodeTables<NC> &t, const float *__restrict__ code) {
    const int tid = threadIdx.x;
    for (int i = tid; i < NC; i += blockDim.x) t.raw[i] = code[i];
    if (tid == 0) { t.lut_bad = 0; t.tiny_thr = 0; }
    __syncthreads();
    // stable rank sort (the reference sorts only when the codebook is not ascending;
    // sorting an ascending codebook is the identity, functional.py:561-565)
    for (int i = tid; i < NC; i += blockDim.x) {
        float v = t.raw[i];
        int rank = 0;
        for (int j = 0; j < NC; ++j) {
            float w = t.raw[j];
            rank += (w < v) || (w == v && j < i);
        }
        t.sorted[rank] = v;
        t.perm[rank] = (unsigned char)i;
    }
    __syncthreads();
    for (int j = tid; j < NC; j += blockDim.x) {
        if (j == NC - 1) { t.thr[j] = CUDART_INF_F; continue; }
        const float lo = t.sorted[j], hi = t.sorted[j + 1];
        // predicate P(q) = |q - lo| > |hi - q| is false at lo and monotone in q
        long long a = float_key(lo), b = float_key(hi);
        if (!(fabsf(hi - lo) > 0.0f)) { t.thr[j] = hi; continue; }
        for (int it = 0; it < 64 && b - a > 1; ++it) {
            long long m = a + ((b - a) >> 1);
            float q = key_float(m);
            bool up = fabsf(q - lo) > fabsf(hi - q);
            if (up) b = m; else a = m;
        }
        t.thr[j] = key_float(b);
        if (fabsf(t.thr[j]) < 8.8817842e-16f) t.tiny_thr = 1;             // 2^-50
    }
    if (tid == 0) {
        bool ident = true;
        for (int j = 0; j < NC; ++j) ident = ident && (t.perm[j] == j);
        t.perm_identity = ident;
        t.cmin = t.sorted[0];
        t.cmax = t.sorted[NC - 1];
        t.need_clamp = !(t.sorted[0] <= -1.0f && t.sorted[NC - 1] >= 1.0f);
    }
    __syncthreads();
    if constexpr (NC == 256) {
        for (int j = tid; j < NC - 1; j += blockDim.x) t.thr_cell[j] = cell8_of(t.thr[j]);   // non-decreasing in j
        __syncthreads();
        for (int k = tid; k <= kCells8; k += blockDim.x) {
            int lo = 0, hi = NC - 1;                          // first threshold whose cell is >= k
            while (lo < hi) { const int mid = (lo + hi) >> 1; if (t.thr_cell[mid] < k) lo = mid + 1; else hi = mid; }
            const int base = lo;
            hi = NC - 1;                                      // first threshold whose cell is > k
            while (lo < hi) { const int mid = (lo + hi) >> 1; if (t.thr_cell[mid] <= k) lo = mid + 1; else hi = mid; }
            t.cell8[k] = (unsigned short)(base | ((lo - base) << 8));
        }
        __syncthreads();
    }
    if (NC == 16) {
        for (int attempt = 0; attempt < 2; ++attempt) {
            const float scale = attempt ? 512.0f : kLutCoarseScale;
            const int last = 2 * (int)scale;                 // highest cell a quotient can reach
            if (tid == 0) { t.lut_bad = 0; t.lut_scale = scale; }
            if (tid < NC - 1) {
                const float th = t.thr[tid];
                int c;
                if (th > 1.0f) c = last + 1;                  // never reached
                else if (!(th >= -1.0f)) c = -1;              // below every quotient
                else {
                    c = lut_cell_raw(th, scale) - 0x4B000000;
                    // the quantizer looks cells up with a quotient that may be 3 ulp off: a threshold
                    // closer than 8 ulp to a cell border would make the neighbouring cell wrong
                    const long long k = float_key(th);
                    if (lut_cell_raw(key_float(k - 8), scale) - 0x4B000000 != c ||
                        lut_cell_raw(key_float(k + 8), scale) - 0x4B000000 != c) t.lut_bad = 1;
                }
                t.thr_cell[tid] = c;
            }
            __syncthreads();
            for (int k = tid; k <= last + 1; k += blockDim.x) {   // cells a finite quotient can index
                int base = 0, inside = 0;
                unsigned thb = 0x7f800000u;                   // +inf: no threshold in this cell
                for (int j = 0; j < NC - 1; ++j) {
                    const int cj = t.thr_cell[j];
                    base += (cj < k);
                    if (cj == k) { ++inside; thb = __float_as_uint(t.thr[j]); }
                }
                if (inside > 1 && k <= last) t.lut_bad = 1;
                t.lut[k] = (thb & ~15u) | (unsigned)min(base, 15);
            }
            __syncthreads();
            if (!t.lut_bad) break;                            // uniform: read after the barrier
            __syncthreads();                                  // everyone has read lut_bad before it is reset
        }
    }
}

// Index of q (|q| <= 1, finite) in the sorted 16-entry codebook through the packed table.
__device__ __forceinline__ int lut_index(const CodeTables<16> &t, const unsigned *lut, float scale, float q) {
    const unsigned e = lut[lut_cell_raw(q, scale) & (kLutAlloc - 1)];
    const int base = (int)(e & 15u);
    int idx = base + (q >= __uint_as_float(e & ~15u) ? 1 : 0);
    // q in the same 16-ulp bucket as the threshold: the cleared bits matter, use the exact value
    if (((__float_as_uint(q) ^ e) & ~15u) == 0u) idx = base + (q >= t.thr[base] ? 1 : 0);
    return idx;
}

// Number of thresholds <= q (== index into the sorted codebook).
template <int NC>
__device__ __forceinline__ int code_index_search(const CodeTables<NC> &t, float q) {
    int lo = 0;
#pragma unroll
    for (int step = NC / 2; step > 0; step >>= 1)
        if (t.thr[lo + step - 1] <= q) lo += step;
    return lo;
}

// x / d rounded to nearest, given r = RN(1/d): one reciprocal multiply and two FMA
// corrections (Markstein).  Exact whenever no intermediate underflows; callers guarantee
// 2^-40 <= d <= 2^60 and treat |quotient| < 2^-60 as "sign only" (see k_quantize_vec).
__device__ __forceinline__ float div_by_recip(float x, float d, float r) {
    float q = x * r;
    q = fmaf(fmaf(-q, d, x), r, q);
    q = fmaf(fmaf(-q, d, x), r, q);
    return q;
}

// Exponent of a scaled fp16 operand plane: with amax = m * 2^k, m in [0.5, 1), e = target - k puts
// the largest scaled entry just below 2^target (0 for an all-zero or non-finite matrix).
__device__ __forceinline__ int exponent_for(float amax, int target) {
    if (!(amax > 0.0f) || !(amax <= 3.0e38f)) return 0;
    int k;
    frexpf(amax, &k);
    return target - k;
}

// Per-lane quantization of EPL elements for every case the lean path of k_quantize_vec does
// not cover (any codebook, clamp, permutation, extreme scales).  Kept out of line on purpose.
// Operands and results travel by value (registers): passing the caller's arrays by reference
// would force them into local memory on the hot path as well.
template <int EPL> struct LaneVals { float v[EPL]; };

template <int NC, int EPL>
__device__ __noinline__ unsigned long long quantize_lane_generic(const CodeTables<NC> &tab, LaneVals<EPL> x, float amax) {
    unsigned long long packed = 0;                        // one byte per element
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        int k = 0;
        if (amax != 0.0f) {
            float q = __fdiv_rn(x.v[j], amax);
            if (tab.need_clamp) q = fminf(fmaxf(q, tab.cmin), tab.cmax);
            int idx;
            if constexpr (NC == 256) {
                // thresholds in lower cells are below q, those in higher cells above it (the cell is
                // monotone in q); only the thresholds of q's own cell are compared
                const unsigned e = tab.cell8[cell8_of(q)];
                const int base = (int)(e & 255u), cnt = (int)(e >> 8);
                idx = base;
                for (int c = 0; c < cnt; ++c) idx += (tab.thr[base + c] <= q) ? 1 : 0;
            } else {
                idx = code_index_search<NC>(tab, q);
            }
            k = tab.perm[idx];
        }
        packed |= (unsigned long long)(unsigned)k << (8 * j);
    }
    return packed;
}

}  // namespace qt
