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
static int g_panel_pairs = 1;                              // measurement hook: 0 = one column per warp at every height
void set_panel_pairs(int on) { g_panel_pairs = on; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Register-resident panel: warp c owns column c, lane l holds rows l, l+32, ... of it for the
// whole factorisation: the first RPL of them in registers, RS more (tall panels only) in the
// column's slots of the shared staging buffer, so that the register budget of a 1024-thread CTA
// (64 per thread) is never exceeded.  Per column step the pivot warp builds its Householder
// vector and publishes it once through a double-buffered shared-memory vector; the warps to
// its right apply the reflector to their own column, the warps to its left (already final)
// take the dot product v_i . v_c needed for the triangular factor T, and warp 0 fills in
// column c-1 of T meanwhile (slarft recurrence), off the critical path.  One barrier per step;
// every reduction chain is split over four accumulators.
//
// Fused form (prev_w > 0): before anything is factored, the block reflector of the PREVIOUS panel
// of the same outer block (Householder vectors in V's columns j0-prev_w .. j0-1, rows j0-prev_w ..
// n-1; its triangular factor Tprev) is applied to 32-column chunks of the rest of the outer block:
//     C <- (I - Vp Tp^T Vp^T) C,   C = A[j0-prev_w : n, j0 + 32 chunk : ...]
// CTA (matrix, chunk) updates chunk `chunk` (written back to A); chunk 0 is the new panel, which
// its CTA goes on to factor from shared memory.  This replaces the three library products per
// panel that a separate rank-32 update needs, and the CTAs of chunks 1.. fill otherwise idle SMs.
template <int RPL, int RS>
__global__ void __launch_bounds__(kQrThreads, 1)
k_householder_panel(float *__restrict__ Abase, long long strideA, int n, int j0, int w,
                    float *__restrict__ Vbase, long long strideV, float *__restrict__ Tbase, long long strideT,
                    int prev_w, const float *__restrict__ Tprev_base, int block_end) {
    constexpr int RT = RPL + RS;
    extern __shared__ float sm[];
    const int m = n - j0;
    float *Pall = sm;                                      // [kPanel + m][33]: rows of the update window, then of the panel
    float *P = Pall + kPanel * 33;                         // [m][33] staging of the panel rows (coalesced global access)
    float *vb = Pall + (((kPanel + m) * 33 + 31) & ~31);   // [2][RT * 32] published Householder vector
    float *G = vb + 2 * RT * 32;                           // [32][33]  v_i . v_j, i < j
    float *Ts = G + kPanel * (kPanel + 1);                 // [32][33]
    float *tau = Ts + kPanel * (kPanel + 1);               // [32]
    float *Vs = tau + kPanel;                              // [256][36] slab of the previous panel's vectors (fused form); later the partial sums of W
    float *Tp = Vs + 256 * 36;                             // [32][33]  previous panel's triangular factor
    float *zs = Tp + kPanel * (kPanel + 1);                // [32][33]  z = Tp^T W
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = blockIdx.y;
    float *Amat = Abase + (long long)blockIdx.x * strideA;
    const float *A = Amat + (long long)j0 * n + j0;

    if (prev_w > 0) {
        // ---- apply the previous panel's block reflector to this CTA's column chunk
        const int r0 = j0 - prev_w;                        // first row of the update window
        const int mu = n - r0;                             // rows of the window
        const int c0 = j0 + kPanel * chunk;                // first column of the chunk
        const int wc = min(kPanel, block_end - c0);        // columns of the chunk
        float *C = Pall + (kPanel - prev_w) * 33;          // window rows so that row prev_w of it is P's row 0
        float *Cg = Amat + (long long)r0 * n + c0;
        const float *Vg = Vbase + (long long)blockIdx.x * strideV + (long long)r0 * n + r0;
        for (int r = warp; r < mu; r += 32) C[r * 33 + lane] = (lane < wc) ? Cg[(long long)r * n + lane] : 0.0f;
        for (int i = tid; i < kPanel * kPanel; i += kQrThreads) {
            const int a = i / kPanel, b = i - a * kPanel;
            Tp[a * (kPanel + 1) + b] = (a < prev_w && b < prev_w) ? Tprev_base[(long long)blockIdx.x * strideT + i] : 0.0f;
        }
        // Vp is streamed through shared memory in slabs of kSlab window rows; the next slab is
        // fetched into registers while the current one is being used, so the global-memory latency
        // of the 2 * ceil(mu / kSlab) dependent slab loads is hidden behind the arithmetic.
        // In both passes a lane works on COLUMN `lane` of the chunk and a warp on a subset of the rows,
        // so a row of Vp is read as broadcast 128-bit loads and serves all 32 columns at once (one
        // warp per column re-read every row 32 times and was bound by shared-memory bandwidth).
        constexpr int kSlab = 256, kVp = 36, kPer = kSlab * kPanel / kQrThreads;    // row pitch 36: 16-byte aligned rows
        float pre[kPer];
        auto fetch = [&](int rb) {
#pragma unroll
            for (int q = 0; q < kPer; ++q) {
                const int i = tid + q * kQrThreads, rr = i >> 5, j = i & 31;
                pre[q] = (rb + rr < mu && j < prev_w) ? Vg[(long long)(rb + rr) * n + j] : 0.0f;
            }
        };
        auto stash = [&]() {
#pragma unroll
            for (int q = 0; q < kPer; ++q) {
                const int i = tid + q * kQrThreads;
                Vs[(i >> 5) * kVp + (i & 31)] = pre[q];
            }
        };
        // ---- W = Vp^T C.  Warp (g, h): reflector columns 8g .. 8g+7, rows h, h+8, .. of each slab.
        const int g8 = (warp >> 3) * 8, h = warp & 7;
        float wacc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) wacc[j] = 0.0f;
        fetch(0);
        for (int rb = 0; rb < mu; rb += kSlab) {
            __syncthreads();
            stash();
            __syncthreads();
            fetch(rb + kSlab < mu ? rb + kSlab : 0);       // after the last slab: the first slab of the second pass
#pragma unroll 4
            for (int k = 0; k < kSlab / 8; ++k) {
                const int rr = h + 8 * k;
                if (rb + rr < mu) {
                    const float cv = C[(rb + rr) * 33 + lane];
                    const float4 v0 = *reinterpret_cast<const float4 *>(Vs + rr * kVp + g8);
                    const float4 v1 = *reinterpret_cast<const float4 *>(Vs + rr * kVp + g8 + 4);
                    wacc[0] = fmaf(v0.x, cv, wacc[0]); wacc[1] = fmaf(v0.y, cv, wacc[1]);
                    wacc[2] = fmaf(v0.z, cv, wacc[2]); wacc[3] = fmaf(v0.w, cv, wacc[3]);
                    wacc[4] = fmaf(v1.x, cv, wacc[4]); wacc[5] = fmaf(v1.y, cv, wacc[5]);
                    wacc[6] = fmaf(v1.z, cv, wacc[6]); wacc[7] = fmaf(v1.w, cv, wacc[7]);
                }
            }
        }
        __syncthreads();                                   // the slab buffer is free: it takes the eight partial sums
        float *Wpart = Vs;                                 // [8 row groups][32][33]
#pragma unroll
        for (int j = 0; j < 8; ++j) Wpart[(h * kPanel + g8 + j) * 33 + lane] = wacc[j];
        __syncthreads();
        float *Wm = G;                                     // [32][33]; G is cleared again before the factorisation
        {
            float wsum = 0.0f;                             // W[warp][lane]
#pragma unroll
            for (int q = 0; q < 8; ++q) wsum += Wpart[(q * kPanel + warp) * 33 + lane];
            Wm[warp * 33 + lane] = wsum;
        }
        __syncthreads();
        {
            float z = 0.0f;                                // z[warp][lane] = (Tp^T W)[warp][lane]
#pragma unroll
            for (int j = 0; j < kPanel; ++j) z = fmaf(Tp[j * (kPanel + 1) + warp], Wm[j * 33 + lane], z);
            zs[warp * 33 + lane] = z;
        }
        __syncthreads();
        float zreg[kPanel];
#pragma unroll
        for (int j = 0; j < kPanel; ++j) zreg[j] = zs[j * 33 + lane];
        // ---- C -= Vp z.  Warp w: rows w, w+32, .. of each slab.
        for (int rb = 0; rb < mu; rb += kSlab) {
            __syncthreads();
            stash();
            __syncthreads();
            if (rb + kSlab < mu) fetch(rb + kSlab);
#pragma unroll 2
            for (int k = 0; k < kSlab / 32; ++k) {
                const int rr = warp + 32 * k;
                if (rb + rr < mu) {
                    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
                    for (int j = 0; j < kPanel; j += 8) {
                        const float4 v0 = *reinterpret_cast<const float4 *>(Vs + rr * kVp + j);
                        const float4 v1 = *reinterpret_cast<const float4 *>(Vs + rr * kVp + j + 4);
                        a0 = fmaf(v0.x, zreg[j], a0); a0 = fmaf(v0.y, zreg[j + 1], a0);
                        a0 = fmaf(v0.z, zreg[j + 2], a0); a0 = fmaf(v0.w, zreg[j + 3], a0);
                        a1 = fmaf(v1.x, zreg[j + 4], a1); a1 = fmaf(v1.y, zreg[j + 5], a1);
                        a1 = fmaf(v1.z, zreg[j + 6], a1); a1 = fmaf(v1.w, zreg[j + 7], a1);
                    }
                    C[(rb + rr) * 33 + lane] -= a0 + a1;
                }
            }
        }
        __syncthreads();
        if (chunk > 0) {                                   // not the new panel: write the updated chunk back and leave
            for (int r = warp; r < mu; r += 32)
                if (lane < wc) Cg[(long long)r * n + lane] = C[r * 33 + lane];
            return;
        }
        // chunk 0: rows prev_w.. of the window are the new panel, already in P
        for (int r = warp; r < m; r += 32)
            if (lane >= w) P[r * 33 + lane] = 0.0f;
    } else {
        for (int r = warp; r < m; r += 32) P[r * 33 + lane] = (lane < w) ? A[(long long)r * n + lane] : 0.0f;
    }
    for (int i = tid; i < 2 * kPanel * (kPanel + 1); i += kQrThreads) G[i] = 0.0f;   // G and Ts are adjacent
    __syncthreads();
    float col[RPL];
#pragma unroll
    for (int k = 0; k < RPL; ++k) {
        const int r = lane + 32 * k;
        col[k] = (r < m) ? P[r * 33 + warp] : 0.0f;
    }
    // element k of this lane's part of the column (k is a compile-time constant after unrolling)
    auto get = [&](int k) -> float {
        if (k < RPL) return col[k < RPL ? k : 0];
        const int r = lane + 32 * k;
        return r < m ? P[r * 33 + warp] : 0.0f;
    };
    auto put = [&](int k, float v) {
        if (k < RPL) { col[k < RPL ? k : 0] = v; return; }
        const int r = lane + 32 * k;
        if (r < m) P[r * 33 + warp] = v;
    };
    // Triangular factor (LAPACK slarft, forward / columnwise): T[:i, i] = -tau_i T[:i, :i] (V^T v_i)[:i].
    // Warp l owns row l of T, lane k holding T[l][k] in a register; column i is added one step after
    // its Gram entries G[:i][i] were written, by all finished warps at once (one product and one warp
    // reduction each), off the critical path of the step.
    // (The tall variants, which keep part of the panel in shared memory, have no register to spare:
    // there warp 0 fills in the column from shared memory as before.)
    constexpr bool T_IN_REGS = RS == 0;
    float trow = 0.0f;
    auto t_column_warp0 = [&](int i) {                      // whole warp; lane l computes T[l][i]
        const float ti = tau[i];
        if (lane == i) Ts[i * (kPanel + 1) + i] = ti;
        if (lane < i) {
            float a0 = 0.0f, a1 = 0.0f;
            int l = lane;
            for (; l + 1 < i; l += 2) {
                a0 = fmaf(Ts[lane * (kPanel + 1) + l], G[l * (kPanel + 1) + i], a0);
                a1 = fmaf(Ts[lane * (kPanel + 1) + l + 1], G[(l + 1) * (kPanel + 1) + i], a1);
            }
            if (l < i) a0 = fmaf(Ts[lane * (kPanel + 1) + l], G[l * (kPanel + 1) + i], a0);
            Ts[lane * (kPanel + 1) + i] = -ti * (a0 + a1);
        }
        __syncwarp();
    };
    auto t_column = [&](int i) {
        if constexpr (!T_IN_REGS) {
            if (warp == 0) t_column_warp0(i);
            return;
        }
        if (warp < i) {
            const float part = (lane >= warp && lane < i) ? trow * G[lane * (kPanel + 1) + i] : 0.0f;
            const float sum = warp_sum(part);
            if (lane == i) trow = -tau[i] * sum;
        } else if (warp == i && lane == i) {
            trow = tau[i];
        }
    };

    for (int c = 0; c < w; ++c) {
        float *vbuf = vb + (c & 1) * (RT * 32);
        if (warp == c) {
            float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int k = 0; k < RT; ++k) {
                const float x = get(k);
                s4[k & 3] = (lane + 32 * k > c) ? fmaf(x, x, s4[k & 3]) : s4[k & 3];
            }
            const float sigma = warp_sum((s4[0] + s4[1]) + (s4[2] + s4[3]));
            const float alpha = __shfl_sync(0xffffffffu, col[0], c);      // row c lives in lane c, slot 0
            float tc = 0.0f, scale = 0.0f;
            if (sigma != 0.0f) {
                const float beta = -copysignf(sqrtf(fmaf(alpha, alpha, sigma)), alpha);
                tc = (beta - alpha) / beta;
                scale = 1.0f / (alpha - beta);
            }
#pragma unroll
            for (int k = 0; k < RT; ++k) {
                const int r = lane + 32 * k;
                const float v = (r > c) ? get(k) * scale : (r == c ? 1.0f : 0.0f);
                put(k, v);                                  // the column now holds v_c (zeros above, one on the diagonal)
                vbuf[k * 32 + lane] = v;
            }
            if (lane == 0) tau[c] = tc;
        }
        __syncthreads();
        if (warp != c && warp < w) {
            float d4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int k = 0; k < RT; ++k) d4[k & 3] = fmaf(vbuf[k * 32 + lane], get(k), d4[k & 3]);
            const float d = warp_sum((d4[0] + d4[1]) + (d4[2] + d4[3]));
            if (warp > c) {                                 // apply H_c = I - tau v v^T to this column
                const float f = tau[c] * d;
#pragma unroll
                for (int k = 0; k < RT; ++k) put(k, fmaf(-f, vbuf[k * 32 + lane], get(k)));
            } else if (lane == 0) {
                G[warp * (kPanel + 1) + c] = d;             // v_warp . v_c
            }
        }
        // column c-1 of T: its dot products were completed before this step's barrier
        if (c >= 1) t_column(c - 1);
    }
    __syncthreads();
    t_column(w - 1);
    if constexpr (T_IN_REGS) Ts[warp * (kPanel + 1) + lane] = (lane >= warp && lane < w && warp < w) ? trow : 0.0f;
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


// Tall panels (more than 640 rows): two columns per warp, 16 warps.  With one column per warp every
// warp reads the whole published Householder vector twice per step and the tall variants also keep
// part of their column in shared memory (64 registers per thread at 1024 threads); here a warp
// reads the vector once for both of its columns and a thread's 2 x RT elements all live in
// registers (128 per thread at 512 threads): a third of the shared-memory traffic per step.
// Warp w owns columns 2w, 2w+1 and rows 2w, 2w+1 of T.  Same conventions, same fused update of the
// previous panel, same outputs as k_householder_panel.
template <int RT>
__global__ void __launch_bounds__(512, 1)
k_householder_panel_pairs(float *__restrict__ Abase, long long strideA, int n, int j0, int w,
                          float *__restrict__ Vbase, long long strideV, float *__restrict__ Tbase, long long strideT,
                          int prev_w, const float *__restrict__ Tprev_base, int block_end) {
    constexpr int NW = 16, NT = NW * 32;
    extern __shared__ float sm[];
    const int m = n - j0;
    float *Pall = sm;                                      // [kPanel + m][33]
    float *P = Pall + kPanel * 33;
    float *vb = Pall + (((kPanel + m) * 33 + 31) & ~31);   // [2][RT * 32] published Householder vector
    float *G = vb + 2 * RT * 32;                           // [32][33]
    float *Ts = G + kPanel * (kPanel + 1);                 // [32][33]
    float *tau = Ts + kPanel * (kPanel + 1);               // [32]
    float *Vs = tau + kPanel;                              // [256][36]
    float *Tp = Vs + 256 * 36;                             // [32][33]
    float *zs = Tp + kPanel * (kPanel + 1);                // [32][33]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = blockIdx.y;
    float *Amat = Abase + (long long)blockIdx.x * strideA;
    const float *A = Amat + (long long)j0 * n + j0;

    if (prev_w > 0) {
        // ---- apply the previous panel's block reflector to this CTA's column chunk
        const int r0 = j0 - prev_w;                        // first row of the update window
        const int mu = n - r0;                             // rows of the window
        const int c0 = j0 + kPanel * chunk;                // first column of the chunk
        const int wc = min(kPanel, block_end - c0);        // columns of the chunk
        float *C = Pall + (kPanel - prev_w) * 33;          // window rows so that row prev_w of it is P's row 0
        float *Cg = Amat + (long long)r0 * n + c0;
        const float *Vg = Vbase + (long long)blockIdx.x * strideV + (long long)r0 * n + r0;
        for (int r = warp; r < mu; r += NW) C[r * 33 + lane] = (lane < wc) ? Cg[(long long)r * n + lane] : 0.0f;
        for (int i = tid; i < kPanel * kPanel; i += NT) {
            const int a = i / kPanel, b = i - a * kPanel;
            Tp[a * (kPanel + 1) + b] = (a < prev_w && b < prev_w) ? Tprev_base[(long long)blockIdx.x * strideT + i] : 0.0f;
        }
        // Vp is streamed through shared memory in slabs of kSlab window rows; the next slab is
        // fetched into registers while the current one is being used, so the global-memory latency
        // of the 2 * ceil(mu / kSlab) dependent slab loads is hidden behind the arithmetic.
        // In both passes a lane works on COLUMN `lane` of the chunk and a warp on a subset of the rows,
        // so a row of Vp is read as broadcast 128-bit loads and serves all 32 columns at once (one
        // warp per column re-read every row 32 times and was bound by shared-memory bandwidth).
        constexpr int kSlab = 256, kVp = 36, kPer = kSlab * kPanel / NT;    // row pitch 36: 16-byte aligned rows
        float pre[kPer];
        auto fetch = [&](int rb) {
#pragma unroll
            for (int q = 0; q < kPer; ++q) {
                const int i = tid + q * NT, rr = i >> 5, j = i & 31;
                pre[q] = (rb + rr < mu && j < prev_w) ? Vg[(long long)(rb + rr) * n + j] : 0.0f;
            }
        };
        auto stash = [&]() {
#pragma unroll
            for (int q = 0; q < kPer; ++q) {
                const int i = tid + q * NT;
                Vs[(i >> 5) * kVp + (i & 31)] = pre[q];
            }
        };
        // ---- W = Vp^T C.  Warp (g, h): reflector columns JG g .. JG g + JG - 1, rows h, h+8, .. of each slab.
        constexpr int JG = kPanel / (NW / 8);
        const int g8 = (warp >> 3) * JG, h = warp & 7;
        float wacc[JG];
#pragma unroll
        for (int j = 0; j < JG; ++j) wacc[j] = 0.0f;
        fetch(0);
        for (int rb = 0; rb < mu; rb += kSlab) {
            __syncthreads();
            stash();
            __syncthreads();
            fetch(rb + kSlab < mu ? rb + kSlab : 0);       // after the last slab: the first slab of the second pass
#pragma unroll 4
            for (int k = 0; k < kSlab / 8; ++k) {
                const int rr = h + 8 * k;
                if (rb + rr < mu) {
                    const float cv = C[(rb + rr) * 33 + lane];
#pragma unroll
                    for (int j = 0; j < JG; j += 4) {
                        const float4 v0 = *reinterpret_cast<const float4 *>(Vs + rr * kVp + g8 + j);
                        wacc[j] = fmaf(v0.x, cv, wacc[j]); wacc[j + 1] = fmaf(v0.y, cv, wacc[j + 1]);
                        wacc[j + 2] = fmaf(v0.z, cv, wacc[j + 2]); wacc[j + 3] = fmaf(v0.w, cv, wacc[j + 3]);
                    }
                }
            }
        }
        __syncthreads();                                   // the slab buffer is free: it takes the eight partial sums
        float *Wpart = Vs;                                 // [8 row groups][32][33]
#pragma unroll
        for (int j = 0; j < JG; ++j) Wpart[(h * kPanel + g8 + j) * 33 + lane] = wacc[j];
        __syncthreads();
        float *Wm = G;                                     // [32][33]; G is cleared again before the factorisation
        for (int jr = warp; jr < kPanel; jr += NW) {
            float wsum = 0.0f;                             // W[jr][lane]
#pragma unroll
            for (int q = 0; q < 8; ++q) wsum += Wpart[(q * kPanel + jr) * 33 + lane];
            Wm[jr * 33 + lane] = wsum;
        }
        __syncthreads();
        for (int jr = warp; jr < kPanel; jr += NW) {
            float z = 0.0f;                                // z[jr][lane] = (Tp^T W)[jr][lane]
#pragma unroll
            for (int j = 0; j < kPanel; ++j) z = fmaf(Tp[j * (kPanel + 1) + jr], Wm[j * 33 + lane], z);
            zs[jr * 33 + lane] = z;
        }
        __syncthreads();
        float zreg[kPanel];
#pragma unroll
        for (int j = 0; j < kPanel; ++j) zreg[j] = zs[j * 33 + lane];
        // ---- C -= Vp z.  Warp w: rows w, w+NW, .. of each slab.
        for (int rb = 0; rb < mu; rb += kSlab) {
            __syncthreads();
            stash();
            __syncthreads();
            if (rb + kSlab < mu) fetch(rb + kSlab);
#pragma unroll 2
            for (int k = 0; k < kSlab / NW; ++k) {
                const int rr = warp + NW * k;
                if (rb + rr < mu) {
                    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
                    for (int j = 0; j < kPanel; j += 8) {
                        const float4 v0 = *reinterpret_cast<const float4 *>(Vs + rr * kVp + j);
                        const float4 v1 = *reinterpret_cast<const float4 *>(Vs + rr * kVp + j + 4);
                        a0 = fmaf(v0.x, zreg[j], a0); a0 = fmaf(v0.y, zreg[j + 1], a0);
                        a0 = fmaf(v0.z, zreg[j + 2], a0); a0 = fmaf(v0.w, zreg[j + 3], a0);
                        a1 = fmaf(v1.x, zreg[j + 4], a1); a1 = fmaf(v1.y, zreg[j + 5], a1);
                        a1 = fmaf(v1.z, zreg[j + 6], a1); a1 = fmaf(v1.w, zreg[j + 7], a1);
                    }
                    C[(rb + rr) * 33 + lane] -= a0 + a1;
                }
            }
        }
        __syncthreads();
        if (chunk > 0) {                                   // not the new panel: write the updated chunk back and leave
            for (int r = warp; r < mu; r += NW)
                if (lane < wc) Cg[(long long)r * n + lane] = C[r * 33 + lane];
            return;
        }
        // chunk 0: rows prev_w.. of the window are the new panel, already in P
        for (int r = warp; r < m; r += NW)
            if (lane >= w) P[r * 33 + lane] = 0.0f;
    } else {
        for (int r = warp; r < m; r += NW) P[r * 33 + lane] = (lane < w) ? A[(long long)r * n + lane] : 0.0f;
    }
    for (int i = tid; i < 2 * kPanel * (kPanel + 1); i += NT) G[i] = 0.0f;   // G and Ts are adjacent
    __syncthreads();
    const int cA = 2 * warp, cB = 2 * warp + 1;
    float colA[RT], colB[RT];
#pragma unroll
    for (int k = 0; k < RT; ++k) {
        const int r = lane + 32 * k;
        colA[k] = (r < m) ? P[r * 33 + cA] : 0.0f;
        colB[k] = (r < m) ? P[r * 33 + cB] : 0.0f;
    }
    float trA = 0.0f, trB = 0.0f;                            // rows cA, cB of T: lane k holds T[row][k]
    auto t_row = [&](int row, float &tr, int i) {
        if (row < i) {
            const float part = (lane >= row && lane < i) ? tr * G[lane * (kPanel + 1) + i] : 0.0f;
            const float sum = warp_sum(part);
            if (lane == i) tr = -tau[i] * sum;
        } else if (row == i && lane == i) {
            tr = tau[i];
        }
    };

    for (int c = 0; c < w; ++c) {
        float *vbuf = vb + (c & 1) * (RT * 32);
        const bool odd = (c & 1) != 0;
        if (warp == (c >> 1)) {
            float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int k = 0; k < RT; ++k) {
                const float x = odd ? colB[k] : colA[k];
                s4[k & 3] = (lane + 32 * k > c) ? fmaf(x, x, s4[k & 3]) : s4[k & 3];
            }
            const float sigma = warp_sum((s4[0] + s4[1]) + (s4[2] + s4[3]));
            const float alpha = __shfl_sync(0xffffffffu, odd ? colB[0] : colA[0], c);   // row c lives in lane c, slot 0
            float tc = 0.0f, scale = 0.0f;
            if (sigma != 0.0f) {
                const float beta = -copysignf(sqrtf(fmaf(alpha, alpha, sigma)), alpha);
                tc = (beta - alpha) / beta;
                scale = 1.0f / (alpha - beta);
            }
#pragma unroll
            for (int k = 0; k < RT; ++k) {
                const int r = lane + 32 * k;
                const float x = odd ? colB[k] : colA[k];
                const float v = (r > c) ? x * scale : (r == c ? 1.0f : 0.0f);
                if (odd) colB[k] = v; else colA[k] = v;      // the column now holds v_c
                vbuf[k * 32 + lane] = v;
            }
            if (lane == 0) tau[c] = tc;
        }
        __syncthreads();
        if (cA < w) {
            float a4[2] = {0.0f, 0.0f}, b4[2] = {0.0f, 0.0f};
#pragma unroll
            for (int k = 0; k < RT; ++k) {
                const float vv = vbuf[k * 32 + lane];
                a4[k & 1] = fmaf(vv, colA[k], a4[k & 1]);
                b4[k & 1] = fmaf(vv, colB[k], b4[k & 1]);
            }
            float dA = a4[0] + a4[1], dB = b4[0] + b4[1];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {         // two reductions interleaved
                dA += __shfl_xor_sync(0xffffffffu, dA, off);
                dB += __shfl_xor_sync(0xffffffffu, dB, off);
            }
            const float tc = tau[c];
            const float fA = (cA > c) ? tc * dA : 0.0f;      // columns to the right of c get H_c applied
            const float fB = (cB > c && cB < w) ? tc * dB : 0.0f;
            if (cB > c) {                                    // at least column B is updated (warp-uniform)
#pragma unroll
                for (int k = 0; k < RT; ++k) {
                    const float vv = vbuf[k * 32 + lane];
                    colA[k] = fmaf(-fA, vv, colA[k]);
                    colB[k] = fmaf(-fB, vv, colB[k]);
                }
            }
            if (lane == 0) {                                 // finished columns: v_col . v_c for the triangular factor
                if (cA < c) G[cA * (kPanel + 1) + c] = dA;
                if (cB < c) G[cB * (kPanel + 1) + c] = dB;
            }
            if (c >= 1) { t_row(cA, trA, c - 1); t_row(cB, trB, c - 1); }
        }
    }
    __syncthreads();
    if (cA < w) { t_row(cA, trA, w - 1); t_row(cB, trB, w - 1); }
    Ts[cA * (kPanel + 1) + lane] = (lane >= cA && lane < w && cA < w) ? trA : 0.0f;
    Ts[cB * (kPanel + 1) + lane] = (lane >= cB && lane < w && cB < w) ? trB : 0.0f;
#pragma unroll
    for (int k = 0; k < RT; ++k) {
        const int r = lane + 32 * k;
        if (r < m) { P[r * 33 + cA] = colA[k]; P[r * 33 + cB] = colB[k]; }
    }
    __syncthreads();
    float *V = Vbase + (long long)blockIdx.x * strideV + (long long)j0 * n + j0;
    for (int r = warp; r < m; r += NW)
        if (lane < w) V[(long long)r * n + lane] = P[r * 33 + lane];
    float *T = Tbase + (long long)blockIdx.x * strideT;
    for (int i = tid; i < kPanel * kPanel; i += NT) T[i] = Ts[(i / kPanel) * (kPanel + 1) + (i % kPanel)];
}

template <int RPL, int RS>
static int launch_panel_rpl(float *A, long long strideA, int n, int count, int j0, int w,
                            float *V, long long strideV, float *T, long long strideT, cudaStream_t s,
                            int prev_w, const float *Tprev, int block_end) {
    const int m = n - j0;
    const size_t smem = sizeof(float) * ((size_t)(((kPanel + m) * 33 + 31) & ~31) + 2 * (RPL + RS) * 32 + 2 * kPanel * (kPanel + 1) + kPanel +
                                         256 * 36 + kPanel * (kPanel + 1) + kPanel * (kPanel + 1));
    static PerDeviceOnce attr_set;                         // function attributes are per device
    const int dev = current_device();
    if (attr_set.pending(dev)) {
        if (cudaFuncSetAttribute(k_householder_panel<RPL, RS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
            return record(QT_ERR_LAUNCH);
        attr_set.mark(dev);
    }
    if (smem > 227 * 1024) return record(QT_ERR_UNSUPPORTED);
    const int chunks = prev_w > 0 ? (block_end - j0 + kPanel - 1) / kPanel : 1;
    dim3 grid(count, chunks);
    k_householder_panel<RPL, RS><<<grid, kQrThreads, smem, s>>>(A, strideA, n, j0, w, V, strideV, T, strideT, prev_w, Tprev, block_end);
    count_launch(1);
    return check_launch();
}

template <int RT>
static int launch_panel_pairs(float *A, long long strideA, int n, int count, int j0, int w,
                              float *V, long long strideV, float *T, long long strideT, cudaStream_t s,
                              int prev_w, const float *Tprev, int block_end) {
    const int m = n - j0;
    const size_t smem = sizeof(float) * ((size_t)(((kPanel + m) * 33 + 31) & ~31) + 2 * RT * 32 + 2 * kPanel * (kPanel + 1) + kPanel +
                                         256 * 36 + kPanel * (kPanel + 1) + kPanel * (kPanel + 1));
    static PerDeviceOnce attr_set;
    const int dev = current_device();
    if (attr_set.pending(dev)) {
        if (cudaFuncSetAttribute(k_householder_panel_pairs<RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
            return record(QT_ERR_LAUNCH);
        attr_set.mark(dev);
    }
    if (smem > 227 * 1024) return record(QT_ERR_UNSUPPORTED);
    const int chunks = prev_w > 0 ? (block_end - j0 + kPanel - 1) / kPanel : 1;
    dim3 grid(count, chunks);
    k_householder_panel_pairs<RT><<<grid, 512, smem, s>>>(A, strideA, n, j0, w, V, strideV, T, strideT, prev_w, Tprev, block_end);
    count_launch(1);
    return check_launch();
}

int launch_householder_panel(float *A, long long strideA, int n, int count, int j0, int w,
                             float *V, long long strideV, float *T, long long strideT, cudaStream_t s,
                             int prev_w, const float *Tprev, int block_end) {
    if (n <= 0 || count < 0 || j0 < 0 || j0 >= n || w <= 0 || w > kPanel || j0 + w > n) return record(QT_ERR_ARG);
    if (!A || !V || !T) return record(QT_ERR_ARG);
    if (prev_w < 0 || prev_w > kPanel || prev_w > j0) return record(QT_ERR_ARG);
    if (prev_w > 0 && (!Tprev || block_end < j0 + w || block_end > n || block_end - j0 > 4 * kPanel)) return record(QT_ERR_ARG);
    if (count == 0) return record(QT_OK);
    if (count > 65535) return record(QT_ERR_UNSUPPORTED);
    const int rows_per_lane = (n - j0 + 31) / 32;
    if (rows_per_lane > kMaxRowsPerLane) return record(QT_ERR_UNSUPPORTED);
#define QT_PANEL(R, S) return launch_panel_rpl<R, S>(A, strideA, n, count, j0, w, V, strideV, T, strideT, s, prev_w, Tprev, block_end)
    if (rows_per_lane <= 6) QT_PANEL(6, 0);
    if (rows_per_lane <= 12) QT_PANEL(12, 0);
    if (rows_per_lane <= 20) QT_PANEL(20, 0);
    if (g_panel_pairs && rows_per_lane > 20) {
        if (rows_per_lane <= 28) return launch_panel_pairs<28>(A, strideA, n, count, j0, w, V, strideV, T, strideT, s, prev_w, Tprev, block_end);
        return launch_panel_pairs<38>(A, strideA, n, count, j0, w, V, strideV, T, strideT, s, prev_w, Tprev, block_end);
    }
    if (rows_per_lane <= 28) QT_PANEL(24, 4);
    QT_PANEL(24, 14);
#undef QT_PANEL
}

// Triangular factor of an outer block of up to four panels from the panels' own factors and
// the Gram matrix G = Vo^T Vo of the block's Householder vectors (LAPACK larft recurrence on
// blocks): with c columns done and the next panel k of width w,
//     T[:c, c:c+w] = -T[:c, :c] * G[:c, c:c+w] * T_k,   T[c:c+w, c:c+w] = T_k.
// One CTA per matrix; T (<= 128 x 128) is assembled in shared memory and written out whole
// (zeros below the diagonal blocks).  Replaces ~17 small library launches per outer block.
static constexpr int kMergeMax = 128;
__global__ void __launch_bounds__(1024)
k_merge_t(const float *__restrict__ Gbase, long long ldg, long long strideG,
          const float *__restrict__ Tp_base, long long strideTp, int wo,
          float *__restrict__ Tbase, long long strideT) {
    extern __shared__ float merge_sm[];
    float (*Ts)[kMergeMax + 1] = reinterpret_cast<float (*)[kMergeMax + 1]>(merge_sm);
    float (*M1)[kPanel + 1] = reinterpret_cast<float (*)[kPanel + 1]>(merge_sm + kMergeMax * (kMergeMax + 1));
    float (*Tk)[kPanel + 1] = reinterpret_cast<float (*)[kPanel + 1]>(merge_sm + kMergeMax * (kMergeMax + 1) + 96 * (kPanel + 1));
    // the Gram matrix is staged once: the recurrence below reads each entry in a dependent chain
    float (*Gs)[kMergeMax + 1] = reinterpret_cast<float (*)[kMergeMax + 1]>(merge_sm + kMergeMax * (kMergeMax + 1) + 96 * (kPanel + 1) +
                                                                            kPanel * (kPanel + 1));
    const float *G = Gbase + (long long)blockIdx.x * strideG;
    const float *Tp = Tp_base + (long long)blockIdx.x * strideTp;
    float *T = Tbase + (long long)blockIdx.x * strideT;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // warp ty works on rows ty, ty+32, ..; lane = column
    for (int i = ty; i < wo; i += 32)
        for (int j = tx; j < wo; j += 32) { Ts[i][j] = 0.0f; Gs[i][j] = __ldg(G + (long long)i * ldg + j); }
    __syncthreads();
    for (int c = 0, k = 0; c < wo; c += kPanel, ++k) {
        const int w = min(kPanel, wo - c);
        Tk[ty][tx] = (ty < w && tx < w) ? Tp[(long long)k * kPanel * kPanel + ty * kPanel + tx] : 0.0f;
        __syncthreads();
        if (ty < w && tx < w) Ts[c + ty][c + tx] = Tk[ty][tx];
        if (c > 0) {
            for (int i = ty; i < c; i += 32) {                   // M1 = T[:c, :c] G[:c, c:c+w]; T is upper triangular
                float acc = 0.0f, acc1 = 0.0f;
                if (tx < w) {
                    int l = i;
                    for (; l + 1 < c; l += 2) {
                        acc = fmaf(Ts[i][l], Gs[l][c + tx], acc);
                        acc1 = fmaf(Ts[i][l + 1], Gs[l + 1][c + tx], acc1);
                    }
                    if (l < c) acc = fmaf(Ts[i][l], Gs[l][c + tx], acc);
                }
                M1[i][tx] = acc + acc1;
            }
            __syncthreads();
            for (int i = ty; i < c; i += 32) {                   // T[:c, c:c+w] = -M1 T_k; T_k is upper triangular
                float acc = 0.0f;
                for (int l = 0; l <= tx; ++l) acc = fmaf(M1[i][l], Tk[l][tx], acc);
                if (tx < w) Ts[i][c + tx] = -acc;
            }
        }
        __syncthreads();
    }
    for (int i = ty; i < wo; i += 32)
        for (int j = tx; j < wo; j += 32) T[(long long)i * wo + j] = Ts[i][j];
}

int launch_merge_t(const float *G, long long ldg, long long strideG, const float *Tp, long long strideTp, int wo, int count,
                   float *T, long long strideT, cudaStream_t s) {
    if (wo <= 0 || wo > kMergeMax || count < 0 || ldg < wo) return record(QT_ERR_ARG);
    if (!G || !Tp || !T) return record(QT_ERR_ARG);
    if (count == 0) return record(QT_OK);
    constexpr size_t smem = sizeof(float) * (2 * kMergeMax * (kMergeMax + 1) + 96 * (kPanel + 1) + kPanel * (kPanel + 1));
    static PerDeviceOnce attr_set;
    const int dev = current_device();
    if (attr_set.pending(dev)) {
        if (cudaFuncSetAttribute(k_merge_t, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return record(QT_ERR_LAUNCH);
        attr_set.mark(dev);
    }
    k_merge_t<<<count, 1024, smem, s>>>(G, ldg, strideG, Tp, strideTp, wo, T, strideT);
    count_launch(1);
    return check_launch();
}

}  // namespace qt
