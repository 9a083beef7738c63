// Batched fp32-accurate matrix products on the 5th-generation tensor cores (tcgen05).
//
// Replaces the fp32 cuBLAS products of the reference's hot path (reference project paths
// optimizers/shampoo2.py:188-199, :265-268; qtensor/utils.py:157-158, :196, :203;
// qtensor/functional.py:757, :762; optimizers/matrix_functions.py:132-135).
//
// Precision scheme ("bf16x3"): every fp32 operand x is carried as two bf16 planes,
// hi = bf16(x) and lo = bf16(x - hi); a product is accumulated in fp32 in tensor memory as
// hi*hi + hi*lo + lo*hi (the lo*lo term, below 2^-16 relative, is dropped).  Three
// tcgen05.mma.kind::f16 instructions per k-slice share one TMEM accumulator.
//
// Kernel structure (persistent: one CTA per SM walks over 128 x 128 output tiles; a ring of TMEM
// accumulators so the epilogue of tile i overlaps the main loop of tile i+1):
//   warp 4      TMA producer: cp.async.bulk.tensor 3-D loads (batch is the third
//               coordinate) of the four operand planes into a 3-stage shared-memory ring,
//               128-byte swizzle, completion on mbarriers;
//   warp 5      allocates the SM's 512 TMEM columns and issues the MMAs (one elected lane);
//               tcgen05.commit releases ring slots and signals the epilogue;
//   warps 0-3   epilogue: tcgen05.ld (32 lanes x 32 columns per instruction), then
//               D = alpha * acc + beta * C in fp32, written as fp32 and/or as bf16 hi/lo
//               planes for the next product of a chain.
// Operands may be K-major (row = M or N index, K contiguous) or MN-major (row = K index).
// Out-of-range rows / columns / k are zero-filled by TMA; the epilogue masks its stores.
// Every wait is bounded: on expiry the kernel records an error word and drains.
#include "quant_device.cuh"
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstring>

namespace qt {

static constexpr int BM = 128, BK = 64;
static constexpr int PLANE_TILE_BYTES = BM * BK * 2;                 // 16 KiB: a 128 x 64 bf16 tile of one plane
static constexpr int RING_BYTES = 12 * PLANE_TILE_BYTES;             // 192 KiB of operand stages
static constexpr int GEMM_SMEM = RING_BYTES + 1024 /*align*/ + 256 /*barriers*/;
static constexpr unsigned WAIT_LIMIT = 1u << 18;

// Tile configuration: NP planes per operand, output tile 128 x BN_.
//   NP = 2, BN_ = 128: 64 KiB per stage, 3 stages   (small problems: more tiles than SMs matter more)
//   NP = 2, BN_ = 256: 96 KiB per stage, 2 stages   (the tensor core reads 12 KiB of operands per
//                      128x256x16 MMA instead of 8 KiB per 128x128x16 one: 25 % less shared-memory
//                      traffic per flop, which is what bounds the 128 x 128 tile)
//   NP = 3, BN_ = 128: 96 KiB per stage, 2 stages
//   PAIR (NP = 2, BN_ = 128): two CTAs of a cluster (an SM pair) share one 256 x 128 tile through
//                      tcgen05 cta_group::2: each CTA stages its own 128 rows of A and only HALF of B
//                      (64 of the 128 columns), 48 KiB per stage instead of 64, 4 stages; the tensor
//                      cores of the pair exchange the B halves between themselves.  25 % less operand
//                      traffic from L2 and from shared memory per flop.
template <int NP, int BN_, int EC, bool CONV = false, bool PAIR = false> struct TileCfg {
    static constexpr int B_PLANE_BYTES = PAIR ? PLANE_TILE_BYTES / 2 : BN_ * BK * 2;   // BN_ rows of 64 k (or BN_ / 64 chunks of 64 x 64)
    static constexpr int STAGE_BYTES = NP * (PLANE_TILE_BYTES + B_PLANE_BYTES);
    static constexpr int STAGES = RING_BYTES / STAGE_BYTES;
    // Epilogue warp e reads TMEM lanes 32 (e & 3) .. +31 and EC accumulator columns starting at
    // EC (e >> 2).  EC = 64 halves the partial sums a thread holds (no register spills with
    // 8 + 2 warps) and doubles the loads in flight for epilogues that stream C, D and planes.
    static constexpr int EPI_WARPS = 4 * (BN_ / EC);
    // CONV: four more warps that build an operand's tiles in shared memory from 4-bit state
    static constexpr int CONV_WARPS = CONV ? 4 : 0;
    static constexpr int THREADS = (EPI_WARPS + 2 + CONV_WARPS) * 32;
    // The whole tensor memory of the SM (one CTA per SM) as a ring of accumulators: four of 128
    // columns, two of 256.  With accumulation chains of 128 k an accumulator is busy for 0.8 us of
    // MMAs only, and the epilogue warps are away for microseconds while they store a finished tile;
    // a ring of two let the MMA issuer run just two chains ahead before it stalled on them.
    static constexpr int TMEM_COLS = 512;
    static constexpr int NACC = TMEM_COLS / BN_;
};

__device__ int g_gemm_error = 0;

// A product operand that lives as 4-bit blockwise state: matrix b of the product is state slot
// slots[b] (null: b); its plane exponent is a_exp[b] / b_exp[b] of GemmParams.
struct QOperand {
    const unsigned char *codes; const float *absmax, *diag; const int *slots;
    long long stride_codes, stride_absmax, stride_diag;                   // per slot: bytes, floats, floats
    int n, nb;                                                            // order of the state matrices, blocks per row
};

struct GemmParams {
    int M, N, K, batch;
    float alpha, beta;
    const float *C; long long ldc, strideC;
    float *D; long long ldd, strideD;
    __nv_bfloat16 *Dhi, *Dmid, *Dlo; long long ldp, strideP;              // result as bf16 planes (Dmid: three-plane kernels)
    __nv_bfloat16 *Thi, *Tmid, *Tlo; float t_c0, t_c1;                    // t_c0 * I + t_c1 * result as three planes
    float *maxdev;                                                        // per matrix: max |result - I| (atomic max)
    const int *a_slot, *b_slot, *d_slot;                                  // per matrix: entry of A / B / outputs (null: the matrix number)
    const int *active;                                                    // per matrix: 0 = skip (null: all)
    // Scaled fp16 planes (two-plane kernels): a plane entry holds value * 2^(exp[entry] + exp0).
    int f16;                                                              // operands and plane outputs are fp16 (else bf16, unscaled)
    const int *a_exp, *b_exp; int ab_exp0;                                // per storage entry exponents of A and B (null: 0) + common part
    const int *out_exp; int *out_exp_w; int out_exp0, out_rel;            // exponent of the plane output: given per entry, or
                                                                          // (out_rel) operand exponents + out_exp0; written to out_exp_w
    int kc;                                                               // k-blocks per accumulation chain (two-plane kernels)
    int c_follows_d;                                                      // C of matrix b is entry d_slot[b] of its array (in-place updates of selected entries)
    // Operands taken straight from 4-bit state (CONV kernels; block size 64, square order qn):
    // codes == nullptr: the operand comes from its planes through TMA as usual.
    QOperand aq, bq;
    const float *oq_code;                                                 // the 16-entry codebook of those operands
    int tiles_m, tiles_n;
    // 4-bit state as C operand and as result (QOUT kernels only): block size 64, order N == M
    const unsigned char *q_in; const float *q_absmax_in, *q_diag_in;      // q_in == nullptr: no C operand
    unsigned char *q_out; float *q_absmax_out, *q_diag_out;                // q_diag_out == nullptr: plain variant
    long long q_stride_codes, q_stride_absmax, q_stride_diag;             // per matrix: bytes, floats, floats
    const float *q_code; int q_nb;
};

// Tile number -> (row band, column band, matrix).  Within a matrix the tiles are walked in groups
// of RASTER_M row bands, column by column, so that the ~148 tiles in flight at any moment form a
// roughly square patch: both operands' k-panels are then shared by a dozen CTAs through L2
// instead of one operand by all and the other by two (matters once a matrix exceeds L2).
static constexpr int RASTER_M = 12;
template <int RASTER = RASTER_M>
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int &tm, int &tn, int &b) {
    const int per_matrix = tiles_m * tiles_n;
    b = tile / per_matrix;
    const int t = tile - b * per_matrix;
    const int group = t / (RASTER * tiles_n);
    const int first_m = group * RASTER;
    const int gsize = min(tiles_m - first_m, RASTER);
    const int r = t - group * RASTER * tiles_n;
    tn = r / gsize;
    tm = first_m + (r - tn * gsize);
}

template <bool Q> struct QuantTablesHolder { CodeTables<16> t; };
template <> struct QuantTablesHolder<false> { int unused; };

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One poll of a barrier's phase.  CLUSTER: acquire at cluster scope (the arrival may come from the
// other CTA of a pair).
template <bool CLUSTER>
__device__ __forceinline__ unsigned mbar_try(unsigned bar, unsigned parity) {
    unsigned ok;
    if constexpr (CLUSTER)
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    else
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded parity wait; also gives up when another role raised the CTA's abort flag.
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int *abort_flag) {
    for (unsigned it = 0; it < WAIT_LIMIT; ++it) {
        const unsigned ok = mbar_try<CLUSTER>(bar, parity);
        if (ok) return true;
        if ((it & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(&g_gemm_error, QT_ERR_TIMEOUT);
    return false;
}
// Warp-collective wait: lane 0 polls with a short sleep between polls (the other 31 lanes and
// the other warps' issue slots stay free for the MMA and TMA threads), result broadcast.
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait_warp(unsigned bar, unsigned parity, volatile int *abort_flag) {
    unsigned ok = 0;
    if ((threadIdx.x & 31) == 0) {
        for (unsigned it = 0; it < WAIT_LIMIT; ++it) {
            ok = mbar_try<CLUSTER>(bar, parity);
            if (ok) break;
            if ((it & 255u) == 255u && *abort_flag) break;
            // try_wait already suspends the thread for a while; an extra sleep only pays once the
            // wait is clearly a long one (an accumulator hand-off every few hundred cycles must not
            // be delayed by a sleep that overshoots)
            if (it > 32u) __nanosleep(20);
        }
        if (!ok && !*abort_flag) {
            *abort_flag = 1;
            atomicExch(&g_gemm_error, QT_ERR_TIMEOUT);
        }
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap *map, unsigned bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
// ---- CTA pairs (cta_group::2) -------------------------------------------------------------
__device__ __forceinline__ unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ unsigned map_to_cta(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Load into this CTA's shared memory; the bytes are counted on a barrier that may belong to the
// other CTA of the pair (`bar`: a shared::cluster address).  No multicast: every CTA fetches its own tile.
__device__ __forceinline__ void tma_load_3d_pair(unsigned dst, const CUtensorMap *map, unsigned bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
// One MMA over both SMs of the pair: 256 x N x 16, rows 0..127 accumulate in this CTA's tensor
// memory, rows 128..255 in the peer's; each CTA's shared memory holds its rows of A and its half of B
// at the offsets the descriptors name.
__device__ __forceinline__ void umma_pair(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                          unsigned idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrival on `bar` (a shared::cluster address, either CTA's) once the pair's MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                          unsigned idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
// 256-bit global accesses (sm_100); addresses must be 32-byte aligned.
__device__ __forceinline__ void ldg256f(const float *p, float *v) {
    asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "l"(p));
}
__device__ __forceinline__ void stg256f(float *p, const float *v) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
}
__device__ __forceinline__ void stg256u(void *p, const unsigned *v) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

__device__ __forceinline__ unsigned long long smem_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// NP = planes per operand: 2 -> hi, lo (three products, ~1e-5); 3 -> hi, mid, lo (six products,
// fp32-level accuracy).  Plane 0 is the most significant one.
struct GemmMaps { CUtensorMap a[3]; CUtensorMap b[3]; };

// Epilogue of the kernels whose C operand and result are 4-bit blockwise state (block 64, packed
// as the stand-alone quantizer packs them).  `sum` holds LEN (64 or 128) consecutive accumulator
// columns of this thread's row starting at column n0, i.e. whole quantization blocks: the old state is dequantized in registers exactly as
// k_dequantize_vec does, combined as beta*old + alpha*sum, and quantized exactly as k_quantize_vec
// does (diagonal side channel, block scale, exact division, threshold table).  The result equals
// quantize(fp32 epilogue output) bit for bit and no fp32 copy of the state touches HBM.
// In-place use (q_out == q_in) is safe: a block's bytes, scale and diagonal entry are read and
// written by this thread only, reads first.
template <int LEN>
__device__ __forceinline__ void quantizing_epilogue(const CodeTables<16> &tab, const GemmParams &p, float (&sum)[LEN],
                                                    int b, int row, int n0, float alpha) {
    const bool lean_launch = !tab.lut_bad && !tab.need_clamp && tab.perm_identity && !tab.tiny_thr;
    const float lut_scale = tab.lut_scale;
#pragma unroll
    for (int h = 0; h < LEN / 64; ++h) {
        const int c0 = n0 + h * 64;
        const int valid = p.N - c0;                            // a multiple of 16 (launcher)
        if (valid <= 0) continue;
        const int blk = c0 >> 6;
        const long long e0 = (long long)row * p.N + c0;        // flat element index, a multiple of 16
        const bool on_diag = (unsigned)(row - c0) < 64u;
        if (p.q_in) {
            const float am = __ldg(p.q_absmax_in + (long long)b * p.q_stride_absmax + (long long)row * p.q_nb + blk);
            const float z = (am == 0.0f) ? 0.0f : -0.0f;       // all-zero block dequantizes to +0.0
            const unsigned char *cin = p.q_in + (long long)b * p.q_stride_codes + (e0 >> 1);
            const bool has_d = p.q_diag_in != nullptr && on_diag;
            const float dold = has_d ? __ldg(p.q_diag_in + (long long)b * p.q_stride_diag + row) : 0.0f;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                if (g * 16 < valid) {
                    const uint2 w = __ldg(reinterpret_cast<const uint2 *>(cin + 8 * g));
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const unsigned byte = ((j < 8 ? w.x : w.y) >> (8 * ((j & 7) >> 1))) & 255u;
                        const unsigned idx = (j & 1) ? (byte & 15u) : (byte >> 4);
                        float old = fmaf(tab.raw[idx], am, z);
                        if (has_d && c0 + g * 16 + j == row) old = dold;
                        sum[h * 64 + g * 16 + j] = fmaf(p.beta, old, alpha * sum[h * 64 + g * 16 + j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) sum[h * 64 + g * 16 + j] = 0.0f;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) sum[h * 64 + j] = (j < valid) ? fmaf(p.beta, 0.0f, alpha * sum[h * 64 + j]) : 0.0f;
        }
        if (p.q_diag_out != nullptr && on_diag) {              // functional.py:574-578
            float dnew = 0.0f;
#pragma unroll
            for (int j = 0; j < 64; ++j)
                if (c0 + j == row) { dnew = sum[h * 64 + j]; sum[h * 64 + j] = 0.0f; }
            p.q_diag_out[(long long)b * p.q_stride_diag + row] = dnew;
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 64; ++j) amax = fmaxf(amax, fabsf(sum[h * 64 + j]));
        p.q_absmax_out[(long long)b * p.q_stride_absmax + (long long)row * p.q_nb + blk] = amax;
        const bool scale_ok = (amax >= 9.094947e-13f && amax <= 1.1529215e18f) || amax == 0.0f;
        const bool lean = lean_launch && scale_ok;
        unsigned char *cout = p.q_out + (long long)b * p.q_stride_codes + (e0 >> 1);
        const float d = (amax == 0.0f) ? 1.0f : amax;
        const float rcp = __frcp_rn(d);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            if (g * 16 >= valid) continue;
            unsigned w0 = 0, w1 = 0;
            if (lean) {
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const int i0 = lut_index(tab, tab.lut, lut_scale, div_by_recip(sum[h * 64 + g * 16 + j], d, rcp));
                    const int i1 = lut_index(tab, tab.lut, lut_scale, div_by_recip(sum[h * 64 + g * 16 + j + 1], d, rcp));
                    const unsigned byte = (unsigned)((i0 << 4) | i1);
                    if (j < 8) w0 |= byte << (4 * j); else w1 |= byte << (4 * (j - 8));
                }
                if (amax == 0.0f) { w0 = 0; w1 = 0; }          // functional.py:600-602
            } else {
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    LaneVals<8> xv;
#pragma unroll
                    for (int j = 0; j < 8; ++j) xv.v[j] = sum[h * 64 + g * 16 + q * 8 + j];
                    const unsigned long long pk = quantize_lane_generic<16, 8>(tab, xv, amax);
                    unsigned w = 0;
#pragma unroll
                    for (int j = 0; j < 8; j += 2)
                        w |= (unsigned)((((pk >> (8 * j)) & 15u) << 4) | ((pk >> (8 * (j + 1))) & 15u)) << (4 * j);
                    if (q == 0) w0 = w; else w1 = w;
                }
            }
            *reinterpret_cast<uint2 *>(cout + 8 * g) = make_uint2(w0, w1);
        }
    }
}

// 16 consecutive result values of one row -> NP bf16 planes (x = hi [+ mid] + lo).  `wide`: one
// 256-bit store per plane (32-byte aligned); otherwise element by element, `nvalid` of them.
template <int NP>
__device__ __forceinline__ void store_planes(__nv_bfloat16 *hi, __nv_bfloat16 *mid, __nv_bfloat16 *lo, const float (&v)[16],
                                             bool wide, int nvalid) {
    unsigned short H[16], M[16], L[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
        const __nv_bfloat16 h = __float2bfloat16_rn(v[t]);
        const float r1 = v[t] - __bfloat162float(h);
        H[t] = __bfloat16_as_ushort(h);
        if constexpr (NP == 3) {
            const __nv_bfloat16 m = __float2bfloat16_rn(r1);
            M[t] = __bfloat16_as_ushort(m);
            L[t] = __bfloat16_as_ushort(__float2bfloat16_rn(r1 - __bfloat162float(m)));
        } else {
            L[t] = __bfloat16_as_ushort(__float2bfloat16_rn(r1));
        }
    }
    if (wide) {
        unsigned w[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = (unsigned)H[2 * t] | ((unsigned)H[2 * t + 1] << 16);
        stg256u(hi, w);
        if constexpr (NP == 3) {
#pragma unroll
            for (int t = 0; t < 8; ++t) w[t] = (unsigned)M[2 * t] | ((unsigned)M[2 * t + 1] << 16);
            stg256u(mid, w);
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = (unsigned)L[2 * t] | ((unsigned)L[2 * t + 1] << 16);
        stg256u(lo, w);
    } else {
#pragma unroll
        for (int t = 0; t < 16; ++t) {
            if (t < nvalid) {
                hi[t] = __ushort_as_bfloat16(H[t]);
                if constexpr (NP == 3) mid[t] = __ushort_as_bfloat16(M[t]);
                lo[t] = __ushort_as_bfloat16(L[t]);
            }
        }
    }
}

// 16 consecutive result values -> two fp16 planes of value * scale (scale a power of two): x = hi + lo
// to 22 significant bits while |x * scale| stays in fp16's normal range.  A value beyond that
// range would turn into inf in the plane: it is clamped and the sticky error word is set.
__device__ __forceinline__ void store_planes_f16(__half *hi, __half *lo, const float (&v)[16], float scale, bool wide, int nvalid) {
    unsigned short H[16], L[16];
    bool bad = false;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
        float x = v[t] * scale;
        if (!(fabsf(x) <= 65000.0f)) { bad = bad || (t < nvalid); x = fminf(fmaxf(x, -65000.0f), 65000.0f); if (!(x == x)) x = 0.0f; }
        const __half h = __float2half_rn(x);
        H[t] = __half_as_ushort(h);
        L[t] = __half_as_ushort(__float2half_rn(x - __half2float(h)));
    }
    if (bad) atomicCAS(&g_gemm_error, 0, QT_ERR_RANGE);
    if (wide) {
        unsigned w[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = (unsigned)H[2 * t] | ((unsigned)H[2 * t + 1] << 16);
        stg256u(hi, w);
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = (unsigned)L[2 * t] | ((unsigned)L[2 * t + 1] << 16);
        stg256u(lo, w);
    } else {
#pragma unroll
        for (int t = 0; t < 16; ++t)
            if (t < nvalid) { hi[t] = __ushort_as_half(H[t]); lo[t] = __ushort_as_half(L[t]); }
    }
}

// 64 consecutive elements of row `row` of a 4-bit state matrix, starting at column `col` (a
// multiple of 64: exactly one quantization block), dequantized exactly as k_dequantize_planes
// does (code * scale, fp32 diagonal restored), scaled by two_e and split into fp16 hi / lo;
// written as eight 16-byte pieces per plane to `dst_hi` / `dst_lo` (shared-memory addresses of
// this row's 128-byte line) with the 128-byte swizzle pattern of line `line` of its 8-line group.
// nvalid: leading elements that exist (a multiple of 16, or 0); the rest is written as zeros.
__device__ __forceinline__ void convert_q4_row(const QOperand &q, const float *code_s, int slot, int row, int col, int nvalid,
                                               float two_e, unsigned dst_hi, unsigned dst_lo, int line) {
    const unsigned char *cp = q.codes + (long long)slot * q.stride_codes + (((long long)row * q.n + col) >> 1);
    float am = 0.0f, dg = 0.0f;
    bool has_d = false;
    if (nvalid > 0) {
        am = __ldg(q.absmax + (long long)slot * q.stride_absmax + (long long)row * q.nb + (col >> 6));
        has_d = q.diag != nullptr && (unsigned)(row - col) < 64u;
        if (has_d) dg = __ldg(q.diag + (long long)slot * q.stride_diag + row);
    }
    const float z = (am == 0.0f) ? 0.0f : -0.0f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {                            // 16 elements (8 code bytes) per step
        uint2 w = make_uint2(0u, 0u);
        const bool live = g * 16 < nvalid;
        if (live) w = __ldg(reinterpret_cast<const uint2 *>(cp + 8 * g));
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {                     // 8 elements -> one 16-byte piece per plane
            unsigned H[4], L[4];
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                const unsigned byte = ((hh ? w.y : w.x) >> (8 * (i >> 1))) & 255u;
                float v0 = fmaf(code_s[byte >> 4], am, z), v1 = fmaf(code_s[byte & 15u], am, z);
                const int c = col + g * 16 + hh * 8 + i;
                if (has_d) { if (c == row) v0 = dg; if (c + 1 == row) v1 = dg; }
                const float a0 = live ? v0 * two_e : 0.0f, a1 = live ? v1 * two_e : 0.0f;
                const __half h0 = __float2half_rn(a0), h1 = __float2half_rn(a1);
                const __half l0 = __float2half_rn(a0 - __half2float(h0)), l1 = __float2half_rn(a1 - __half2float(h1));
                H[i >> 1] = (unsigned)__half_as_ushort(h0) | ((unsigned)__half_as_ushort(h1) << 16);
                L[i >> 1] = (unsigned)__half_as_ushort(l0) | ((unsigned)__half_as_ushort(l1) << 16);
            }
            const unsigned off = (unsigned)(((g * 2 + hh) ^ (line & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst_hi + off), "r"(H[0]), "r"(H[1]), "r"(H[2]), "r"(H[3]) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst_lo + off), "r"(L[0]), "r"(L[1]), "r"(L[2]), "r"(L[3]) : "memory");
        }
    }
}

template <bool A_MN, bool B_MN, int NP, int BN_, int EC, bool QOUT = false, bool CONV = false, bool PAIR = false>
__global__ void __launch_bounds__(TileCfg<NP, BN_, EC, CONV, PAIR>::THREADS, 1)
k_gemm_bf16x3(const __grid_constant__ GemmMaps maps, const GemmParams p) {
    using Cfg = TileCfg<NP, BN_, EC, CONV, PAIR>;
    static_assert(!CONV || (NP == 2 && !A_MN && B_MN && BN_ == 128), "operands from 4-bit state: A row-major, B row-major, two planes");
    static_assert(!PAIR || (NP == 2 && BN_ == 128 && !CONV && !QOUT), "CTA pairs: plain two-plane products with 128-column tiles");
    // PAIR: launched as clusters of two CTAs.  CTA rank r of a pair owns rows [128 r, +128) of the
    // pair's 256 x 128 tile and columns [64 r, +64) of its B operand.  Rank 0 (the leader) issues
    // the MMAs for both; every CTA runs its own TMA producer and epilogue.  p.tiles_m counts
    // 256-row bands.  Barrier traffic between the two CTAs:
    //   full[s]      leader's only: counts the TMA bytes of BOTH CTAs;
    //   empty[s]     one per CTA, both signalled by the leader's tcgen05.commit;
    //   acc_full[a]  one per CTA, both signalled by the leader's tcgen05.commit;
    //   acc_empty[a] leader's only: the epilogue warps of both CTAs arrive on it.
    // Waits stay bounded; a CTA never returns before the final cluster barrier, so its peer never
    // touches shared or tensor memory of a CTA that is gone.
    const unsigned rank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = rank == 0u;
    const int cta_first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;     // first tile of this CTA (pair)
    const int cta_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    constexpr int TILE_M = PAIR ? 2 * BM : BM;
    __shared__ float conv_code[CONV ? 16 : 1];
    __shared__ QuantTablesHolder<QOUT> qtab;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int EPI_WARPS = Cfg::EPI_WARPS;
    constexpr int B_PLANE_BYTES = Cfg::B_PLANE_BYTES;
    // The tensor core's fp32 accumulation truncates: the error of one accumulation chain grows
    // linearly with its length (measured 6.5e-9 * K relative, biased).  The three-plane variant
    // therefore accumulates at most KC k-blocks (128 k) per TMEM accumulator and the epilogue
    // warps add the partial sums in fp32 registers (round to nearest) while the next chunk is
    // being multiplied; the two-plane variant, whose operands carry 16 significant bits anyway,
    // runs one chain per tile when its operands are bf16 planes (16 significant bits: the
    // operand rounding dominates anyway) and chains of p.kc k-blocks when they are scaled fp16
    // planes (22 bits).
    const int KC = NP == 3 ? 2 : (p.kc > 0 ? p.kc : (1 << 20));
    extern __shared__ unsigned char smem_raw[];
    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *aligned = smem_raw + (base - smem_u32(smem_raw));
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(aligned + RING_BYTES);
    // bars[0..S): full, [S..2S): empty, [2S..2S+NACC): accumulator full, [2S+NACC..2S+2 NACC): accumulator empty
    constexpr int NACC = Cfg::NACC;
    unsigned *tmem_slot = reinterpret_cast<unsigned *>(bars + 2 * STAGES + 2 * NACC);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const unsigned bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto acc_full = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
    auto acc_empty = [&](int a) { return bar0 + 8u * (2 * STAGES + NACC + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // a wait that expired in an earlier CTA (or launch) poisons the rest of the grid: drain fast
    // (not in a pair: the two CTAs could decide differently, and one would wait for the other)
    if (!PAIR && *reinterpret_cast<volatile int *>(&g_gemm_error) != 0) return;
    const int num_kb = (p.K + BK - 1) / BK;
    const int num_tiles = p.tiles_m * p.tiles_n * p.batch;
    const int nchunks = (num_kb + KC - 1) / KC;

    const bool conv_a = CONV && p.aq.codes != nullptr, conv_b = CONV && p.bq.codes != nullptr;
    if (threadIdx.x == 0) {
        // a stage is full when the TMA bytes have landed and, for an operand built from 4-bit
        // state, when each of the four converter warps has arrived
        const unsigned full_count = 1u + ((conv_a || conv_b) ? (unsigned)Cfg::CONV_WARPS : 0u);
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), full_count); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < NACC; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), PAIR ? 2 * EPI_WARPS : EPI_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == EPI_WARPS + 1) {
        if constexpr (PAIR) {
            // the same warp of both CTAs allocates the same columns in both tensor memories
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();                   // the peer's barriers are initialised, its tensor memory allocated
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_slot;
    if constexpr (QOUT) build_tables<16>(qtab.t, p.q_code);    // all threads; ends with a barrier
    if constexpr (CONV) {
        if (threadIdx.x < 16 && p.oq_code) conv_code[threadIdx.x] = p.oq_code[threadIdx.x];
        __syncthreads();
    }

    // A matrix whose entry of `active` is zero is skipped by all three roles alike (the array
    // does not change while the kernel runs), so their ring and accumulator counters stay in step.
    auto skipped = [&](int b) { return p.active != nullptr && __ldg(p.active + b) == 0; };

    if (warp == EPI_WARPS) {
        // ---------------- TMA producer: one ring of stages shared by all tiles of this CTA
        if (lane == 0) {
            unsigned it = 0;
            bool ok = true;
            for (int tile = cta_first; tile < num_tiles && ok; tile += cta_step) {
                int tm, tn, b;
                tile_coords<PAIR ? RASTER_M / 2 : RASTER_M>(tile, p.tiles_m, p.tiles_n, tm, tn, b);
                if (skipped(b)) continue;
                const int za = p.a_slot ? __ldg(p.a_slot + b) : b;
                const int zb = p.b_slot ? __ldg(p.b_slot + b) : b;
                const int m0 = tm * TILE_M + (int)rank * BM, n0 = tn * BN_;
                // pair: this CTA stages the columns [n0 + rank * ncur / 2, + ncur / 2) of B (ncur: the
                // tile's existing columns rounded up to 16, as the MMA issuer computes it)
                const int nhalf = min(BN_, (p.N - n0 + 15) & ~15) >> 1;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait<PAIR>(empty_bar(s), ((it / STAGES) & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    const unsigned stage = base + s * STAGE_BYTES;
                    const int k0 = kb * BK;
                    if constexpr (PAIR) {
                        const unsigned lead_full = map_to_cta(full_bar(s), 0u);
                        if (leader) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
#pragma unroll
                        for (int pl = 0; pl < NP; ++pl) {
                            const unsigned ta = stage + pl * PLANE_TILE_BYTES;
                            const unsigned tb = stage + NP * PLANE_TILE_BYTES + pl * B_PLANE_BYTES;
                            if (!A_MN) {
                                tma_load_3d_pair(ta, &maps.a[pl], lead_full, k0, m0, za);
                            } else {
                                tma_load_3d_pair(ta, &maps.a[pl], lead_full, m0, k0, za);
                                tma_load_3d_pair(ta + PLANE_TILE_BYTES / 2, &maps.a[pl], lead_full, m0 + 64, k0, za);
                            }
                            if (!B_MN) tma_load_3d_pair(tb, &maps.b[pl], lead_full, k0, n0 + (int)rank * nhalf, zb);
                            else       tma_load_3d_pair(tb, &maps.b[pl], lead_full, n0 + (int)rank * nhalf, k0, zb);
                        }
                        continue;
                    }
                    mbar_expect_tx(full_bar(s), STAGE_BYTES - (conv_a ? NP * PLANE_TILE_BYTES : 0) - (conv_b ? NP * B_PLANE_BYTES : 0));
#pragma unroll
                    for (int pl = 0; pl < NP; ++pl) {
                        const unsigned ta = stage + pl * PLANE_TILE_BYTES;
                        const unsigned tb = stage + NP * PLANE_TILE_BYTES + pl * B_PLANE_BYTES;
                        if (conv_a) {
                        } else if (!A_MN) {
                            tma_load_3d(ta, &maps.a[pl], full_bar(s), k0, m0, za);
                        } else {
                            tma_load_3d(ta, &maps.a[pl], full_bar(s), m0, k0, za);
                            tma_load_3d(ta + PLANE_TILE_BYTES / 2, &maps.a[pl], full_bar(s), m0 + 64, k0, za);
                        }
                        if (conv_b) {
                        } else if (!B_MN) {
                            tma_load_3d(tb, &maps.b[pl], full_bar(s), k0, n0, zb);
                        } else {
#pragma unroll
                            for (int c = 0; c < BN_ / 64; ++c)
                                tma_load_3d(tb + c * (PLANE_TILE_BYTES / 2), &maps.b[pl], full_bar(s), n0 + 64 * c, k0, zb);
                        }
                    }
                }
            }
        }
    } else if (warp == EPI_WARPS + 1) {
        // ---------------- MMA issuer: accumulator j % NACC in TMEM columns [ (j % NACC) * BN_, +BN_ )
        if (lane == 0 && leader) {
            // instruction descriptor: fp32 accumulate, bf16 x bf16, majors, N, M (256 for a CTA pair)
            const unsigned fmt = p.f16 ? 0u : ((1u << 7) | (1u << 10));          // operand format: 0 = fp16, 1 = bf16
            const unsigned idesc = (1u << 4) | fmt | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                   ((unsigned)(BN_ >> 3) << 17) | ((unsigned)(TILE_M >> 4) << 24);
            // descriptors differ only in their 14-bit start-address field: build one per operand
            // plane for stage 0, k-slice 0 and add (byte offset >> 4) afterwards
            const unsigned a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u;
            unsigned long long dA[NP], dB[NP];
#pragma unroll
            for (int pl = 0; pl < NP; ++pl) {
                dA[pl] = smem_desc(base + pl * PLANE_TILE_BYTES, a_lbo, 1024u);
                dB[pl] = smem_desc(base + NP * PLANE_TILE_BYTES + pl * B_PLANE_BYTES, b_lbo, 1024u);
            }
            constexpr unsigned a_step = (A_MN ? 2048u : 32u) >> 4, b_step = (B_MN ? 2048u : 32u) >> 4;
            unsigned it = 0;
            bool ok = true;
            int j = 0;                                      // accumulator hand-offs so far
            for (int tile = cta_first; tile < num_tiles && ok; tile += cta_step) {
                // a ragged last column band needs only its own columns (N is any multiple of 16):
                // the tensor core's time per MMA scales with N
                int tm_, tn_, b_;
                tile_coords<PAIR ? RASTER_M / 2 : RASTER_M>(tile, p.tiles_m, p.tiles_n, tm_, tn_, b_);
                if (skipped(b_)) continue;
                const int ncur = min(BN_, (p.N - tn_ * BN_ + 15) & ~15);
                const unsigned idesc_tile = (idesc & ~(0x3Fu << 17)) | ((unsigned)(ncur >> 3) << 17);
                int kb = 0;
                for (int ch = 0; ch < nchunks && ok; ++ch, ++j) {
                    const int acc = j % NACC;
                    ok = mbar_wait<PAIR>(acc_empty(acc), ((j / NACC) & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned tmem_acc = tmem_base + (unsigned)(acc * BN_);
                    const int kend = min(num_kb, kb + KC);
                    for (bool fresh = true; kb < kend; ++kb, ++it, fresh = false) {
                        const int s = it % STAGES;
                        ok = mbar_wait<PAIR>(full_bar(s), (it / STAGES) & 1, abort_flag);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        // K-major: 8-row groups 1024 B apart, a 16-element k-slice is 32 B further along the row.
                        // MN-major: 64-wide MN chunks 8192 B apart (LBO), 8-k-row groups 1024 B apart, a k-slice is 2048 B further.
                        const unsigned long long soff = (unsigned long long)((unsigned)(s * STAGE_BYTES) >> 4);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k) {
                            const unsigned long long ao = soff + k * a_step, bo = soff + k * b_step;
                            // every pair of planes whose combined significance is above the dropped
                            // residual: index sum <= NP - 1, least significant pairs first
                            bool first = fresh && k == 0;
#pragma unroll
                            for (int sum = NP - 1; sum >= 0; --sum) {
#pragma unroll
                                for (int ia = 0; ia <= sum; ++ia) {
                                    if constexpr (PAIR) umma_pair(tmem_acc, dA[ia] + ao, dB[sum - ia] + bo, idesc_tile, first ? 0u : 1u);
                                    else                umma_bf16(tmem_acc, dA[ia] + ao, dB[sum - ia] + bo, idesc_tile, first ? 0u : 1u);
                                    first = false;
                                }
                            }
                        }
                        if constexpr (PAIR) {                      // the slot is free in both CTAs
                            umma_commit_pair(empty_bar(s));
                            umma_commit_pair(map_to_cta(empty_bar(s), 1u));
                        } else {
                            umma_commit(empty_bar(s));
                        }
                    }
                    if (ok) {
                        if constexpr (PAIR) {                      // both CTAs' epilogues read their half of the rows
                            umma_commit_pair(acc_full(acc));
                            umma_commit_pair(map_to_cta(acc_full(acc), 1u));
                        } else {
                            umma_commit(acc_full(acc));
                        }
                    }
                }
            }
        }
    } else if (warp < EPI_WARPS) {
        // ---------------- epilogue: warp e reads TMEM lanes 32 (e & 3) .. +31 (lane = output row) and
        // the 128 accumulator columns [128 (e >> 2), +128) of the tile.  Partial sums of the chunks
        // are added in registers; the final combine / conversion / store works on 16 columns at a
        // time with 256-bit accesses straight from registers (no shared-memory staging: the tensor
        // core's operand fetch already uses the shared-memory bandwidth).
        const int quad = warp & 3, seg = warp >> 2;
        const bool has_c = p.C != nullptr && p.beta != 0.0f;
        const bool wide_d = ((p.ldc | p.ldd | p.strideC | p.strideD) & 7) == 0 &&
                            ((reinterpret_cast<uintptr_t>(p.C) | reinterpret_cast<uintptr_t>(p.D)) & 31) == 0;
        const bool wide_p = ((p.ldp | p.strideP) & 15) == 0 &&
                            ((reinterpret_cast<uintptr_t>(p.Dhi) | reinterpret_cast<uintptr_t>(p.Dmid) | reinterpret_cast<uintptr_t>(p.Dlo) |
                              reinterpret_cast<uintptr_t>(p.Thi) | reinterpret_cast<uintptr_t>(p.Tmid) | reinterpret_cast<uintptr_t>(p.Tlo)) & 31) == 0;
        int j = 0;
        const unsigned lead_acc_empty0 = PAIR ? map_to_cta(acc_empty(0), 0u) : 0u;
        for (int tile = cta_first; tile < num_tiles; tile += cta_step) {
            int tm, tn, b;
            tile_coords<PAIR ? RASTER_M / 2 : RASTER_M>(tile, p.tiles_m, p.tiles_n, tm, tn, b);
            if (skipped(b)) continue;
            if constexpr (PAIR) tm = 2 * tm + (int)rank;       // this CTA's 128-row band
            const int m0 = tm * BM, n0 = tn * BN_ + seg * EC;
            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            const int valid = min(EC, p.N - n0);               // columns of this warp's segment that exist (may be <= 0)
            float sum[EC];
#pragma unroll
            for (int q = 0; q < EC; ++q) sum[q] = 0.0f;
            bool ok = true;
            for (int ch = 0; ch < nchunks; ++ch, ++j) {
                const int acc = j % NACC;
                ok = mbar_wait_warp<PAIR>(acc_full(acc), (j / NACC) & 1, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned tmem_acc = tmem_base + (unsigned)(acc * BN_ + seg * EC);
                if (valid > 0) {
#pragma unroll
                    for (int c = 0; c < EC / 32; ++c) {
                        float v[32];
                        tmem_ld32(tmem_acc + ((unsigned)(quad * 32) << 16) + (unsigned)(c * 32), v);
#pragma unroll
                        for (int q = 0; q < 32; ++q) sum[c * 32 + q] += v[q];
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    if constexpr (PAIR) mbar_arrive_cluster(lead_acc_empty0 + 8u * acc);
                    else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(acc)) : "memory");
                }
            }
            if (!ok) break;
            // scaled operand planes: the accumulator holds sum(a * 2^ea * b * 2^eb)
            int e_in = 0;
            if (p.f16) {
                const int za = p.a_slot ? __ldg(p.a_slot + b) : b, zb = p.b_slot ? __ldg(p.b_slot + b) : b;
                e_in = (p.a_exp ? __ldg(p.a_exp + za) : 0) + (p.b_exp ? __ldg(p.b_exp + zb) : 0) + p.ab_exp0;
            }
            const float alpha_eff = p.f16 ? p.alpha * exp2f((float)-e_in) : p.alpha;
            if constexpr (QOUT) {
                if (row_ok && valid > 0) quantizing_epilogue<EC>(qtab.t, p, sum, b, row, n0, alpha_eff);
            } else {
                const int bo = p.d_slot ? __ldg(p.d_slot + b) : b;
                float dev = 0.0f;                               // max |result - I| over this thread's elements
                float pscale = 1.0f;                            // plane entry = value * pscale (fp16 planes)
                if (p.f16 && p.Dhi) {
                    const int e_out = p.out_exp ? __ldg(p.out_exp + bo) + p.out_exp0 : (p.out_rel ? e_in + p.out_exp0 : p.out_exp0);
                    pscale = exp2f((float)e_out);
                    if (p.out_exp_w && tm == 0 && tn == 0 && seg == 0 && quad == 0 && lane == 0) p.out_exp_w[bo] = e_out;
                }
                if (row_ok && valid > 0) {
                    const float *crow = p.C + (long long)(p.c_follows_d ? bo : b) * p.strideC + (long long)row * p.ldc + n0;
                    float *drow = p.D + (long long)bo * p.strideD + (long long)row * p.ldd + n0;
                    const long long po = (long long)bo * p.strideP + (long long)row * p.ldp + n0;
                    const long long to = (long long)b * p.strideP + (long long)row * p.ldp + n0;   // T is stored by matrix number
                    // C is fetched two 16-column groups ahead of its use (the two-plane tiles; one group
                    // ahead where 128 partial sums leave no registers): a product with a short K and a C
                    // operand is bound by this stream, and eight warps with one 64-byte request each in
                    // flight keep an SM at half of its share of the HBM bandwidth
                    constexpr int CPF = (EC <= 64 && !CONV) ? 2 : 1;
                    float cnext[CPF][16];
                    auto fetch_c = [&](int q, float (&dst)[16]) {
                        if (!has_c || q >= valid) return;
                        if (q + 16 <= valid && wide_d) { ldg256f(crow + q, dst); ldg256f(crow + q + 8, dst + 8); }
                        else {
#pragma unroll
                            for (int t = 0; t < 16; ++t) dst[t] = (q + t < valid) ? __ldg(crow + q + t) : 0.0f;
                        }
                    };
                    fetch_c(0, cnext[0]);
                    if constexpr (CPF == 2) fetch_c(16, cnext[1]);
#pragma unroll
                    for (int q = 0; q < EC; q += 16) {
                        if (q >= valid) continue;
                        const bool full16 = q + 16 <= valid;
                        float o[16];
                        if (has_c) {
#pragma unroll
                            for (int t = 0; t < 16; ++t) o[t] = cnext[(q >> 4) % CPF][t];
                            if (q + 16 * CPF < EC) fetch_c(q + 16 * CPF, cnext[(q >> 4) % CPF]);
#pragma unroll
                            for (int t = 0; t < 16; ++t) o[t] = fmaf(p.beta, o[t], alpha_eff * sum[q + t]);
                        } else {
#pragma unroll
                            for (int t = 0; t < 16; ++t) o[t] = alpha_eff * sum[q + t];
                        }
                        if (p.D) {
                            if (full16 && wide_d) { stg256f(drow + q, o); stg256f(drow + q + 8, o + 8); }
                            else {
#pragma unroll
                                for (int t = 0; t < 16; ++t) if (q + t < valid) drow[q + t] = o[t];
                            }
                        }
                        if (p.Dhi) {
                            if (NP == 2 && p.f16)
                                store_planes_f16(reinterpret_cast<__half *>(p.Dhi) + po + q, reinterpret_cast<__half *>(p.Dlo) + po + q, o,
                                                 pscale, full16 && wide_p, valid - q);
                            else
                                store_planes<NP>(p.Dhi + po + q, NP == 3 ? p.Dmid + po + q : nullptr, p.Dlo + po + q, o,
                                                 full16 && wide_p, valid - q);
                        }
                        if (p.maxdev || p.Thi) {
                            const int dcol = row - (n0 + q);    // position of the diagonal inside this group, if any
                            if (p.maxdev) {
#pragma unroll
                                for (int t = 0; t < 16; ++t) {
                                    if (q + t < valid) {
                                        float a = fabsf(o[t] - (t == dcol ? 1.0f : 0.0f));
                                        if (!(a <= 3.0e38f)) a = CUDART_INF_F;     // NaN or inf: never "converged"
                                        dev = fmaxf(dev, a);
                                    }
                                }
                            }
                            if (p.Thi) {
                                float tv[16];
#pragma unroll
                                for (int t = 0; t < 16; ++t) tv[t] = fmaf(p.t_c1, o[t], t == dcol ? p.t_c0 : 0.0f);
                                store_planes<3>(p.Thi + to + q, p.Tmid + to + q, p.Tlo + to + q, tv, full16 && wide_p, valid - q);
                            }
                        }
                    }
                }
                if (p.maxdev) {
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) dev = fmaxf(dev, __shfl_xor_sync(0xffffffffu, dev, off));
                    if (lane == 0 && dev > 0.0f) atomicMax(reinterpret_cast<int *>(p.maxdev + b), __float_as_int(dev));
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    } else if (CONV && (conv_a || conv_b)) {
        // ---------------- converter warps: the operand that lives as 4-bit state is dequantized
        // here, straight into the swizzled tile the tensor core reads - the state's fp32 form and
        // its operand planes never exist in device memory.  Thread t builds one 128-byte line:
        // A (row-major, K contiguous): tile row t, the quantization block at columns k0 .. k0+63;
        // B (row-major, N contiguous): k-row t & 63 of the 64-column chunk t >> 6.
        const int t = threadIdx.x - (EPI_WARPS + 2) * 32;
        unsigned it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int tm, tn, b;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn, b);
            if (skipped(b)) continue;
            const int m0 = tm * BM, n0 = tn * BN_;
            const int sa = conv_a ? (p.aq.slots ? __ldg(p.aq.slots + b) : b) : 0;
            const int sb = conv_b ? (p.bq.slots ? __ldg(p.bq.slots + b) : b) : 0;
            const float ea = conv_a ? exp2f((float)(p.a_exp ? __ldg(p.a_exp + b) : 0)) : 1.0f;
            const float eb = conv_b ? exp2f((float)(p.b_exp ? __ldg(p.b_exp + b) : 0)) : 1.0f;
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % STAGES;
                ok = mbar_wait_warp(empty_bar(s), ((it / STAGES) & 1) ^ 1, abort_flag);
                if (!ok) break;
                const unsigned stage = base + s * STAGE_BYTES;
                const int k0 = kb * BK;
                if (conv_a) {
                    const int row = m0 + t;
                    const int nvalid = row < p.M ? max(0, min(64, p.K - k0)) : 0;
                    const unsigned line = stage + (unsigned)t * 128u;
                    convert_q4_row(p.aq, conv_code, sa, row, k0, nvalid, ea, line, line + PLANE_TILE_BYTES, t);
                }
                if (conv_b) {
                    const int kr = t & 63, chunk = t >> 6;
                    const int krow = k0 + kr, col = n0 + 64 * chunk;
                    const int nvalid = krow < p.K ? max(0, min(64, p.N - col)) : 0;
                    const unsigned line = stage + NP * PLANE_TILE_BYTES + (unsigned)chunk * (PLANE_TILE_BYTES / 2) + (unsigned)kr * 128u;
                    convert_q4_row(p.bq, conv_code, sb, krow, col, nvalid, eb, line, line + B_PLANE_BYTES, kr);
                }
                // make the generic-proxy writes visible to the tensor core's (async-proxy) reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full_bar(s)) : "memory");
            }
        }
    }
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();                   // neither CTA frees or leaves while its peer still works
    if (warp == EPI_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
    }
}

// fp32 -> (hi, lo) bf16 planes.  Vector variant: 8 consecutive elements per thread (two 128-bit
// loads, two 128-bit stores); scalar variant for unaligned or ragged rows.
__device__ __forceinline__ void split2(float a, float b, unsigned &h, unsigned &l) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(a), h1 = __float2bfloat16_rn(b);
    const __nv_bfloat16 l0 = __float2bfloat16_rn(a - __bfloat162float(h0));
    const __nv_bfloat16 l1 = __float2bfloat16_rn(b - __bfloat162float(h1));
    h = (unsigned)__bfloat16_as_ushort(h0) | ((unsigned)__bfloat16_as_ushort(h1) << 16);
    l = (unsigned)__bfloat16_as_ushort(l0) | ((unsigned)__bfloat16_as_ushort(l1) << 16);
}

__global__ void __launch_bounds__(256)
k_split_bf16_vec(const float *__restrict__ X, long long ldx, long long strideX, int rows, int cols8,
                 __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo, long long ldp, long long strideP) {
    const int b = blockIdx.y;
    const float *x = X + (long long)b * strideX;
    __nv_bfloat16 *h = hi + (long long)b * strideP, *l = lo + (long long)b * strideP;
    const long long total = (long long)rows * cols8;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(e / cols8), c = (int)(e - (long long)r * cols8) * 8;
        const float4 v0 = __ldg(reinterpret_cast<const float4 *>(x + (long long)r * ldx + c));
        const float4 v1 = __ldg(reinterpret_cast<const float4 *>(x + (long long)r * ldx + c + 4));
        uint4 H, L;
        split2(v0.x, v0.y, H.x, L.x); split2(v0.z, v0.w, H.y, L.y);
        split2(v1.x, v1.y, H.z, L.z); split2(v1.z, v1.w, H.w, L.w);
        *reinterpret_cast<uint4 *>(h + (long long)r * ldp + c) = H;
        *reinterpret_cast<uint4 *>(l + (long long)r * ldp + c) = L;
    }
}

// 16 elements per thread with 256-bit accesses (two loads, one store per plane); needs 32-byte
// aligned rows in the source and in both planes.
__global__ void __launch_bounds__(256)
k_split_bf16_wide(const float *__restrict__ X, long long ldx, long long strideX, int rows, int cols16,
                  __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo, long long ldp, long long strideP) {
    const int b = blockIdx.y;
    const float *x = X + (long long)b * strideX;
    __nv_bfloat16 *h = hi + (long long)b * strideP, *l = lo + (long long)b * strideP;
    const long long total = (long long)rows * cols16;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(e / cols16), c = (int)(e - (long long)r * cols16) * 16;
        float v[16];
        ldg256f(x + (long long)r * ldx + c, v);
        ldg256f(x + (long long)r * ldx + c + 8, v + 8);
        unsigned H[8], L[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) split2(v[2 * j], v[2 * j + 1], H[j], L[j]);
        stg256u(h + (long long)r * ldp + c, H);
        stg256u(l + (long long)r * ldp + c, L);
    }
}

// Split with a row gather and / or a row scale: output row i of matrix b is
// scale[b][i] * X[b][index[b][i]][:] (either may be absent).  This folds the row selection of the kept
// eigenvectors and the diag(w) factor of rows^T diag(w) rows into the operand preparation.
// WIDE: 16 elements per thread with 256-bit accesses; otherwise one element per thread.
template <bool WIDE>
__global__ void __launch_bounds__(256)
k_split_bf16_rows(const float *__restrict__ X, long long ldx, long long strideX, int rows, int cols,
                  const long long *__restrict__ index, long long stride_index,
                  const float *__restrict__ scale, long long stride_scale,
                  __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo, long long ldp, long long strideP) {
    const int b = blockIdx.y;
    const float *x = X + (long long)b * strideX;
    __nv_bfloat16 *h = hi + (long long)b * strideP, *l = lo + (long long)b * strideP;
    const long long *idx = index ? index + (long long)b * stride_index : nullptr;
    const float *sc = scale ? scale + (long long)b * stride_scale : nullptr;
    constexpr int E = WIDE ? 16 : 1;
    const int per_row = cols / E;
    const long long total = (long long)rows * per_row;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(e / per_row), c = (int)(e - (long long)r * per_row) * E;
        const long long src = idx ? idx[r] : (long long)r;
        const float f = sc ? sc[r] : 1.0f;
        if constexpr (WIDE) {
            float v[16];
            ldg256f(x + src * ldx + c, v);
            ldg256f(x + src * ldx + c + 8, v + 8);
            unsigned H[8], L[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) split2(sc ? f * v[2 * j] : v[2 * j], sc ? f * v[2 * j + 1] : v[2 * j + 1], H[j], L[j]);
            stg256u(h + (long long)r * ldp + c, H);
            stg256u(l + (long long)r * ldp + c, L);
        } else {
            float v = x[src * ldx + c];
            if (sc) v *= f;
            const __nv_bfloat16 vh = __float2bfloat16_rn(v);
            h[(long long)r * ldp + c] = vh;
            l[(long long)r * ldp + c] = __float2bfloat16_rn(v - __bfloat162float(vh));
        }
    }
}

__global__ void __launch_bounds__(256)
k_split_bf16(const float *__restrict__ X, long long ldx, long long strideX, int rows, int cols,
             __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo, long long ldp, long long strideP) {
    const int b = blockIdx.y;
    const float *x = X + (long long)b * strideX;
    __nv_bfloat16 *h = hi + (long long)b * strideP, *l = lo + (long long)b * strideP;
    const long long total = (long long)rows * cols;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(e / cols), c = (int)(e - (long long)r * cols);
        const float v = x[(long long)r * ldx + c];
        const __nv_bfloat16 vh = __float2bfloat16_rn(v);
        h[(long long)r * ldp + c] = vh;
        l[(long long)r * ldp + c] = __float2bfloat16_rn(v - __bfloat162float(vh));
    }
}

// ------------------------------------------------------------------------------------
// Scaled fp16 planes.  For every matrix b of a batch the largest magnitude amax[b] of the
// (optionally row-gathered, row-scaled) source is found first; the exponent e[b] = target - k with
// amax = m * 2^k, m in [0.5, 1) puts the largest scaled entry just below 2^target, and the planes
// hold hi = fp16(x * 2^e), lo = fp16(x * 2^e - hi): 22 significant bits for every entry within
// 2^(target + 3) of the largest one and an absolute error below 2^-25 (scaled) for the rest.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_amax_rows(const float *__restrict__ X, long long ldx, long long strideX, int rows, int cols,
            const long long *__restrict__ index, long long stride_index,
            const float *__restrict__ scale, long long stride_scale, float *__restrict__ amax) {
    const int b = blockIdx.y;
    const float *x = X + (long long)b * strideX;
    const long long *idx = index ? index + (long long)b * stride_index : nullptr;
    const float *sc = scale ? scale + (long long)b * stride_scale : nullptr;
    const bool vec = (cols & 3) == 0 && (ldx & 3) == 0 && (strideX & 3) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0;
    const int per_row = vec ? cols / 4 : cols;
    const long long total = (long long)rows * per_row;
    float m = 0.0f;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(e / per_row), c = (int)(e - (long long)r * per_row);
        const long long src = idx ? idx[r] : (long long)r;
        const float f = sc ? fabsf(sc[r]) : 1.0f;
        if (vec) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(x + src * ldx + 4 * c));
            m = fmaxf(m, f * fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        } else {
            m = fmaxf(m, f * fabsf(x[src * ldx + c]));
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(reinterpret_cast<int *>(amax + b), __float_as_int(m));
}

// fp32 -> scaled fp16 planes with optional row gather / row scale (see k_split_bf16_rows).
// The exponent comes from amax[b] (then it is also written to exp_out[b]) or, when amax is
// null, from exp_in[b] (null: 0); `target` / `exp0` is added as described above.
template <bool WIDE>
__global__ void __launch_bounds__(256)
k_split_f16_rows(const float *__restrict__ X, long long ldx, long long strideX, int rows, int cols,
                 const long long *__restrict__ index, long long stride_index,
                 const float *__restrict__ scale, long long stride_scale,
                 const float *__restrict__ amax, const int *__restrict__ exp_in, int target_or_exp0, int *__restrict__ exp_out,
                 __half *__restrict__ hi, __half *__restrict__ lo, long long ldp, long long strideP) {
    const int b = blockIdx.y;
    const float *x = X + (long long)b * strideX;
    __half *h = hi + (long long)b * strideP, *l = lo + (long long)b * strideP;
    const long long *idx = index ? index + (long long)b * stride_index : nullptr;
    const float *sc = scale ? scale + (long long)b * stride_scale : nullptr;
    const int e = amax ? exponent_for(amax[b], target_or_exp0) : (exp_in ? exp_in[b] : 0) + target_or_exp0;
    if (exp_out && blockIdx.x == 0 && threadIdx.x == 0) exp_out[b] = e;
    const float two_e = exp2f((float)e);
    constexpr int E = WIDE ? 16 : 1;
    const int per_row = cols / E;
    const long long total = (long long)rows * per_row;
    float worst = 0.0f;                                      // a bound the caller vouched for may be violated
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(t / per_row), c = (int)(t - (long long)r * per_row) * E;
        const long long src = idx ? idx[r] : (long long)r;
        const float f = (sc ? sc[r] : 1.0f) * two_e;
        if constexpr (WIDE) {
            float v[16];
            ldg256f(x + src * ldx + c, v);
            ldg256f(x + src * ldx + c + 8, v + 8);
            unsigned H[8], L[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float a0 = fminf(fmaxf(v[2 * j] * f, -65000.0f), 65000.0f), a1 = fminf(fmaxf(v[2 * j + 1] * f, -65000.0f), 65000.0f);
                worst = fmaxf(worst, fmaxf(fabsf(a0), fabsf(a1)));
                const __half h0 = __float2half_rn(a0), h1 = __float2half_rn(a1);
                const __half l0 = __float2half_rn(a0 - __half2float(h0)), l1 = __float2half_rn(a1 - __half2float(h1));
                H[j] = (unsigned)__half_as_ushort(h0) | ((unsigned)__half_as_ushort(h1) << 16);
                L[j] = (unsigned)__half_as_ushort(l0) | ((unsigned)__half_as_ushort(l1) << 16);
            }
            stg256u(h + (long long)r * ldp + c, H);
            stg256u(l + (long long)r * ldp + c, L);
        } else {
            const float a = fminf(fmaxf(x[src * ldx + c] * f, -65000.0f), 65000.0f);
            worst = fmaxf(worst, fabsf(a));
            const __half vh = __float2half_rn(a);
            h[(long long)r * ldp + c] = vh;
            l[(long long)r * ldp + c] = __float2half_rn(a - __half2float(vh));
        }
    }
    if (worst >= 65000.0f) atomicCAS(&g_gemm_error, 0, QT_ERR_RANGE);
}

// amax (float, batch entries): scratch that receives each matrix's largest magnitude (compute_amax)
// or per-matrix upper bounds the caller already knows; exp_out receives the exponents.
int launch_split_f16(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                     const long long *index, long long stride_index, const float *scale, long long stride_scale,
                     float *amax, int compute_amax, const int *exp_in, int target_or_exp0, int *exp_out,
                     void *hi, void *lo, long long ldp, long long strideP, cudaStream_t s) {
    if (rows < 0 || cols < 0 || batch < 0 || batch > 65535) return record(QT_ERR_ARG);
    if (rows == 0 || cols == 0 || batch == 0) return record(QT_OK);
    if (!X || !hi || !lo || ldx < cols || ldp < cols) return record(QT_ERR_ARG);
    const bool wide = cols % 16 == 0 && ldx % 8 == 0 && strideX % 8 == 0 && ldp % 16 == 0 && strideP % 16 == 0 &&
                      ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 31) == 0;
    const long long total = (long long)rows * (wide ? cols / 16 : cols);
    long long ctas = (total + 256 * 4 - 1) / (256 * 4);
    const long long cap = ((long long)device_sm_count() * 32 + batch - 1) / batch;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    dim3 grid((unsigned)ctas, batch);
    if (amax && compute_amax) {
        if (cudaMemsetAsync(amax, 0, sizeof(float) * batch, s) != cudaSuccess) return record(QT_ERR_LAUNCH);
        k_amax_rows<<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols, index, stride_index, scale, stride_scale, amax);
        count_launch(1);
    }
    if (wide)
        k_split_f16_rows<true><<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols, index, stride_index, scale, stride_scale,
                                                     amax, exp_in, target_or_exp0, exp_out, static_cast<__half *>(hi), static_cast<__half *>(lo), ldp, strideP);
    else
        k_split_f16_rows<false><<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols, index, stride_index, scale, stride_scale,
                                                      amax, exp_in, target_or_exp0, exp_out, static_cast<__half *>(hi), static_cast<__half *>(lo), ldp, strideP);
    count_launch(1);
    return check_launch();
}

// ------------------------------------------------------------------------------------
// Host side.
// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// Plane of a logical (outer x inner) bf16 matrix per batch entry, `ld` elements between rows.
static bool make_map(CUtensorMap *map, const void *base, long long inner, long long outer, long long batch,
                     long long ld, long long stride_batch, unsigned box_inner, unsigned box_outer, bool f16 = false) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)stride_batch * 2};
    cuuint32_t box[3] = {box_inner, box_outer, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_split_bf16(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                      void *hi, void *lo, long long ldp, long long strideP, cudaStream_t s) {
    if (rows < 0 || cols < 0 || batch < 0 || batch > 65535) return record(QT_ERR_ARG);
    if (rows == 0 || cols == 0 || batch == 0) return record(QT_OK);
    if (!X || !hi || !lo || ldx < cols || ldp < cols) return record(QT_ERR_ARG);
    const bool vec = cols % 8 == 0 && ldx % 4 == 0 && strideX % 4 == 0 && ldp % 8 == 0 && strideP % 8 == 0 &&
                     (reinterpret_cast<uintptr_t>(X) & 15) == 0 && (reinterpret_cast<uintptr_t>(hi) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(lo) & 15) == 0;
    const bool wide = vec && cols % 16 == 0 && ldx % 8 == 0 && strideX % 8 == 0 && ldp % 16 == 0 && strideP % 16 == 0 &&
                      (reinterpret_cast<uintptr_t>(X) & 31) == 0 && (reinterpret_cast<uintptr_t>(hi) & 31) == 0 &&
                      (reinterpret_cast<uintptr_t>(lo) & 31) == 0;
    const long long total = wide ? (long long)rows * (cols / 16) : vec ? (long long)rows * (cols / 8) : (long long)rows * cols;
    long long ctas = (total + 256 * 4 - 1) / (256 * 4);
    const long long cap = (148LL * 32 + batch - 1) / batch;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    dim3 grid((unsigned)ctas, batch);
    if (wide)
        k_split_bf16_wide<<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols / 16, static_cast<__nv_bfloat16 *>(hi),
                                                static_cast<__nv_bfloat16 *>(lo), ldp, strideP);
    else if (vec)
        k_split_bf16_vec<<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols / 8, static_cast<__nv_bfloat16 *>(hi),
                                               static_cast<__nv_bfloat16 *>(lo), ldp, strideP);
    else
        k_split_bf16<<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols, static_cast<__nv_bfloat16 *>(hi),
                                           static_cast<__nv_bfloat16 *>(lo), ldp, strideP);
    count_launch(1);
    return check_launch();
}

// fp32 -> three bf16 planes (hi, mid, lo): x = hi + mid + lo to 24 bits.
// Three planes, 16 elements per thread with 256-bit accesses (32-byte aligned rows everywhere).
__global__ void __launch_bounds__(256)
k_split_bf16_3_wide(const float *__restrict__ X, long long ldx, long long strideX, int rows, int cols16,
                    __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ mid, __nv_bfloat16 *__restrict__ lo,
                    long long ldp, long long strideP) {
    const int b = blockIdx.y;
    const float *x = X + (long long)b * strideX;
    const long long po = (long long)b * strideP;
    const long long total = (long long)rows * cols16;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(e / cols16), c = (int)(e - (long long)r * cols16) * 16;
        float v[16];
        ldg256f(x + (long long)r * ldx + c, v);
        ldg256f(x + (long long)r * ldx + c + 8, v + 8);
        unsigned H[8], M[8], L[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            unsigned short hh[2], mm[2], ll[2];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const float a = v[2 * j + t];
                const __nv_bfloat16 h = __float2bfloat16_rn(a);
                const float r1 = a - __bfloat162float(h);
                const __nv_bfloat16 m = __float2bfloat16_rn(r1);
                hh[t] = __bfloat16_as_ushort(h);
                mm[t] = __bfloat16_as_ushort(m);
                ll[t] = __bfloat16_as_ushort(__float2bfloat16_rn(r1 - __bfloat162float(m)));
            }
            H[j] = (unsigned)hh[0] | ((unsigned)hh[1] << 16);
            M[j] = (unsigned)mm[0] | ((unsigned)mm[1] << 16);
            L[j] = (unsigned)ll[0] | ((unsigned)ll[1] << 16);
        }
        const long long o = po + (long long)r * ldp + c;
        stg256u(hi + o, H);
        stg256u(mid + o, M);
        stg256u(lo + o, L);
    }
}

__global__ void __launch_bounds__(256)
k_split_bf16_3(const float *__restrict__ X, long long ldx, long long strideX, int rows, int cols,
               __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ mid, __nv_bfloat16 *__restrict__ lo,
               long long ldp, long long strideP) {
    const int b = blockIdx.y;
    const float *x = X + (long long)b * strideX;
    const long long po = (long long)b * strideP;
    const long long total = (long long)rows * cols;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(e / cols), c = (int)(e - (long long)r * cols);
        const float v = x[(long long)r * ldx + c];
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        const float r1 = v - __bfloat162float(h);
        const __nv_bfloat16 m = __float2bfloat16_rn(r1);
        const long long o = po + (long long)r * ldp + c;
        hi[o] = h; mid[o] = m; lo[o] = __float2bfloat16_rn(r1 - __bfloat162float(m));
    }
}

int launch_split_bf16_rows(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                           const long long *index, long long stride_index, const float *scale, long long stride_scale,
                           void *hi, void *lo, long long ldp, long long strideP, cudaStream_t s) {
    if (rows < 0 || cols < 0 || batch < 0 || batch > 65535) return record(QT_ERR_ARG);
    if (rows == 0 || cols == 0 || batch == 0) return record(QT_OK);
    if (!X || !hi || !lo || ldx < cols || ldp < cols) return record(QT_ERR_ARG);
    const bool wide = cols % 16 == 0 && ldx % 8 == 0 && strideX % 8 == 0 && ldp % 16 == 0 && strideP % 16 == 0 &&
                      ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 31) == 0;
    const long long total = (long long)rows * (wide ? cols / 16 : cols);
    long long ctas = (total + 256 * 4 - 1) / (256 * 4);
    const long long cap = (148LL * 32 + batch - 1) / batch;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    dim3 grid((unsigned)ctas, batch);
    if (wide)
        k_split_bf16_rows<true><<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols, index, stride_index, scale, stride_scale,
                                                      static_cast<__nv_bfloat16 *>(hi), static_cast<__nv_bfloat16 *>(lo), ldp, strideP);
    else
        k_split_bf16_rows<false><<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols, index, stride_index, scale, stride_scale,
                                                       static_cast<__nv_bfloat16 *>(hi), static_cast<__nv_bfloat16 *>(lo), ldp, strideP);
    count_launch(1);
    return check_launch();
}

int launch_split_bf16_3(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                        void *hi, void *mid, void *lo, long long ldp, long long strideP, cudaStream_t s) {
    if (rows < 0 || cols < 0 || batch < 0 || batch > 65535) return record(QT_ERR_ARG);
    if (rows == 0 || cols == 0 || batch == 0) return record(QT_OK);
    if (!X || !hi || !mid || !lo || ldx < cols || ldp < cols) return record(QT_ERR_ARG);
    const bool wide = cols % 16 == 0 && ldx % 8 == 0 && strideX % 8 == 0 && ldp % 16 == 0 && strideP % 16 == 0 &&
                      ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(mid) |
                        reinterpret_cast<uintptr_t>(lo)) & 31) == 0;
    long long ctas = ((long long)rows * (wide ? cols / 16 : cols) + 1023) / 1024;
    const long long cap = (148LL * 32 + batch - 1) / batch;
    if (ctas > cap) ctas = cap;
    dim3 grid((unsigned)(ctas < 1 ? 1 : ctas), batch);
    if (wide) {
        k_split_bf16_3_wide<<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols / 16, static_cast<__nv_bfloat16 *>(hi),
                                                  static_cast<__nv_bfloat16 *>(mid), static_cast<__nv_bfloat16 *>(lo), ldp, strideP);
        count_launch(1);
        return check_launch();
    }
    k_split_bf16_3<<<grid, 256, 0, s>>>(X, ldx, strideX, rows, cols, static_cast<__nv_bfloat16 *>(hi),
                                         static_cast<__nv_bfloat16 *>(mid), static_cast<__nv_bfloat16 *>(lo), ldp, strideP);
    count_launch(1);
    return check_launch();
}

struct GemmArgs {
    const void *Ahi, *Alo; long long lda, strideA; int a_mn;
    const void *Bhi, *Blo; long long ldb, strideB; int b_mn;
    int M, N, K, batch; float alpha, beta;
    const float *C; long long ldc, strideC;
    float *D; long long ldd, strideD;
    void *Dhi, *Dlo; long long ldp, strideP;
};

// Optional extras of a product (all pointers device memory, any of them may be null).
struct GemmExtras {
    void *Dmid = nullptr;                                   // middle result plane (three-plane products)
    void *Thi = nullptr, *Tmid = nullptr, *Tlo = nullptr;   // t_c0 * I + t_c1 * result, three planes (pitch of the result planes)
    float t_c0 = 0.0f, t_c1 = 0.0f;
    float *maxdev = nullptr;                                // per matrix max |result - I|
    const int *a_slot = nullptr, *b_slot = nullptr, *d_slot = nullptr;
    const int *active = nullptr;
    int a_entries = 0, b_entries = 0;                       // matrices in A's / B's storage (0: batch)
    // scaled fp16 planes (two-plane products only)
    int f16 = 0;
    const int *a_exp = nullptr, *b_exp = nullptr; int ab_exp0 = 0;
    const int *out_exp = nullptr; int *out_exp_w = nullptr; int out_exp0 = 0, out_rel = 0;
    int kc = 0;                                             // k-blocks per accumulation chain (0: one chain)
    // operands straight from 4-bit state (see QOperand); codes == nullptr: from planes
    QOperand aq = {nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0}, bq = {nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0};
    const float *oq_code = nullptr;
    int max_ctas = 0;                                       // > 0: cap of the persistent grid (SMs left to kernels on other streams)
    int c_follows_d = 0;                                    // C indexed through d_slot like the outputs
};

static inline bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// 4-bit state operands of the quantizing variant (all device pointers; see GemmParams).
struct QuantStateArgs {
    const float *code;
    const unsigned char *q_in; const float *absmax_in, *diag_in;
    unsigned char *q_out; float *absmax_out, *diag_out;
    long long stride_codes, stride_absmax, stride_diag;
};

typedef void (*GemmKern)(const GemmMaps, const GemmParams);

// Kernel table: [tile configuration][A major][B major][quantizing epilogue].
// Configurations: 0 = two planes, 128 x 128 tile, eight epilogue warps of 64 columns; 1 = two planes, 128 x 256,
// eight epilogue warps of 128 columns; 2 = three planes, 128 x 128, four epilogue warps.
template <int NP, int BN_, int EC> static void fill_kernels(GemmKern (&t)[2][2][2]) {
    t[0][0][0] = k_gemm_bf16x3<false, false, NP, BN_, EC, false>; t[0][0][1] = k_gemm_bf16x3<false, false, NP, BN_, EC, true>;
    t[0][1][0] = k_gemm_bf16x3<false, true, NP, BN_, EC, false>;  t[0][1][1] = k_gemm_bf16x3<false, true, NP, BN_, EC, true>;
    t[1][0][0] = k_gemm_bf16x3<true, false, NP, BN_, EC, false>;  t[1][0][1] = k_gemm_bf16x3<true, false, NP, BN_, EC, true>;
    t[1][1][0] = k_gemm_bf16x3<true, true, NP, BN_, EC, false>;   t[1][1][1] = k_gemm_bf16x3<true, true, NP, BN_, EC, true>;
}
static GemmKern g_kernels[6][2][2][2];
static const int g_cfg_threads[6] = {TileCfg<2, 128, 64>::THREADS, TileCfg<2, 256, 128>::THREADS, TileCfg<3, 128, 128>::THREADS,
                                     TileCfg<2, 128, 64, true>::THREADS, TileCfg<2, 128, 64, false, true>::THREADS,
                                     TileCfg<2, 192, 96>::THREADS};
static const int g_cfg_bn[6] = {128, 256, 128, 128, 128, 192};

static bool prepare_kernels() {
    static bool filled = false;
    if (!filled) {
        fill_kernels<2, 128, 64>(g_kernels[0]);
        fill_kernels<2, 256, 128>(g_kernels[1]);
        fill_kernels<3, 128, 128>(g_kernels[2]);
        // configuration 3: operands from 4-bit state (row-major A and B only)
        for (int i = 0; i < 8; ++i) g_kernels[3][(i >> 2) & 1][(i >> 1) & 1][i & 1] = nullptr;
        g_kernels[3][0][1][0] = k_gemm_bf16x3<false, true, 2, 128, 64, false, true>;
        // configuration 4: CTA pairs (cta_group::2) on 256 x 128 tiles, plain epilogue only
        for (int i = 0; i < 8; ++i) g_kernels[4][(i >> 2) & 1][(i >> 1) & 1][i & 1] = nullptr;
        g_kernels[4][0][0][0] = k_gemm_bf16x3<false, false, 2, 128, 64, false, false, true>;
        g_kernels[4][0][1][0] = k_gemm_bf16x3<false, true, 2, 128, 64, false, false, true>;
        g_kernels[4][1][0][0] = k_gemm_bf16x3<true, false, 2, 128, 64, false, false, true>;
        g_kernels[4][1][1][0] = k_gemm_bf16x3<true, true, 2, 128, 64, false, false, true>;
        // configuration 5: 128 x 192 tiles, eight epilogue warps of 96 columns, plain epilogue only
        for (int i = 0; i < 8; ++i) g_kernels[5][(i >> 2) & 1][(i >> 1) & 1][i & 1] = nullptr;
        g_kernels[5][0][0][0] = k_gemm_bf16x3<false, false, 2, 192, 96>;
        g_kernels[5][0][1][0] = k_gemm_bf16x3<false, true, 2, 192, 96>;
        g_kernels[5][1][0][0] = k_gemm_bf16x3<true, false, 2, 192, 96>;
        g_kernels[5][1][1][0] = k_gemm_bf16x3<true, true, 2, 192, 96>;
        filled = true;
    }
    static PerDeviceOnce attr_done;                      // function attributes are per device
    const int dev = current_device();
    if (attr_done.pending(dev)) {
        for (int i = 0; i < 48; ++i) {
            GemmKern k = g_kernels[i / 8][(i >> 2) & 1][(i >> 1) & 1][i & 1];
            if (k && cudaFuncSetAttribute(reinterpret_cast<const void *>(k), cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM) != cudaSuccess)
                return false;
        }
        attr_done.mark(dev);
    }
    return true;
}

// Test hook: tile configuration of two-plane products.  -1: chosen by problem size (128 x 192 for
// products wider than 128 columns with at least 256 k, else 128 x 128); 128 / 192 / 256: single CTAs
// with that tile width; 512: CTA pairs wherever they are possible.
static int g_force_bn = -1;

// a.Ahi/Alo (+ Amid/Bmid for three planes: order hi, mid, lo).  With `qs` the result (and the C
// operand, if qs->q_in) is 4-bit state instead of a.C / a.D.
int launch_gemm_planes(const GemmArgs &a, const void *Amid, const void *Bmid, cudaStream_t s, const QuantStateArgs *qs,
                       const GemmExtras *ex = nullptr) {
    const int np = (Amid && Bmid) ? 3 : 2;
    static const GemmExtras none;
    const GemmExtras &x = ex ? *ex : none;
    if (qs) {
        if (a.M != a.N || a.N % 16 != 0) return record(QT_ERR_UNSUPPORTED);
        if (!qs->code || !qs->q_out || !qs->absmax_out) return record(QT_ERR_ARG);
        if (qs->q_in && !qs->absmax_in) return record(QT_ERR_ARG);
        // 8-byte code words per 16 elements
        if ((reinterpret_cast<uintptr_t>(qs->q_out) | reinterpret_cast<uintptr_t>(qs->q_in)) & 7) return record(QT_ERR_ARG);
        if (a.batch > 1 && (qs->stride_codes & 7)) return record(QT_ERR_ARG);
    }
    if (a.M < 0 || a.N < 0 || a.K < 0 || a.batch < 0) return record(QT_ERR_ARG);
    if (a.M == 0 || a.N == 0 || a.batch == 0) return record(QT_OK);
    if (a.K == 0) return record(QT_ERR_UNSUPPORTED);
    const bool qa = x.aq.codes != nullptr, qb = x.bq.codes != nullptr;
    if (qa || qb) {
        // operands from 4-bit state: scaled fp16 two-plane products with row-major operands only
        if (np != 2 || !x.f16 || a.a_mn || !a.b_mn || qs || !x.oq_code) return record(QT_ERR_UNSUPPORTED);
        if (qa && (x.aq.n != a.M || a.K != a.M || x.aq.n % 16 || !x.aq.absmax || !x.a_exp)) return record(QT_ERR_ARG);
        if (qb && (x.bq.n != a.N || a.K != a.N || x.bq.n % 16 || !x.bq.absmax || !x.b_exp)) return record(QT_ERR_ARG);
        if ((qa && ((reinterpret_cast<uintptr_t>(x.aq.codes) & 7) || (x.aq.stride_codes & 7))) ||
            (qb && ((reinterpret_cast<uintptr_t>(x.bq.codes) & 7) || (x.bq.stride_codes & 7)))) return record(QT_ERR_ARG);
    }
    if ((!qa && (!a.Ahi || !a.Alo)) || (!qb && (!a.Bhi || !a.Blo)) || (!qs && !a.D && !a.Dhi && !x.Thi && !x.maxdev)) return record(QT_ERR_ARG);
    if ((a.Dhi == nullptr) != (a.Dlo == nullptr) || (Amid == nullptr) != (Bmid == nullptr)) return record(QT_ERR_ARG);
    if (a.Dhi && np == 3 && !x.Dmid) return record(QT_ERR_ARG);                  // three-plane result needs all three planes
    if (x.Thi && (!x.Tmid || !x.Tlo || np != 3 || a.ldp <= 0)) return record(QT_ERR_ARG);
    if ((x.Thi || x.maxdev || x.Dmid) && qs) return record(QT_ERR_UNSUPPORTED);
    if (x.f16 && np != 2) return record(QT_ERR_UNSUPPORTED);
    if (x.kc < 0) return record(QT_ERR_ARG);
    const int a_entries = x.a_entries > 0 ? x.a_entries : a.batch, b_entries = x.b_entries > 0 ? x.b_entries : a.batch;
    const void *Ap[3] = {a.Ahi, np == 3 ? Amid : a.Alo, a.Alo};
    const void *Bp[3] = {a.Bhi, np == 3 ? Bmid : a.Blo, a.Blo};
    // TMA: 16-byte aligned bases, row pitches and batch strides
    for (int i = 0; i < np; ++i)
        if ((!qa && !al16(Ap[i])) || (!qb && !al16(Bp[i]))) return record(QT_ERR_ARG);
    if ((!qa && (a.lda % 8 || a.strideA % 8)) || (!qb && (a.ldb % 8 || a.strideB % 8))) return record(QT_ERR_ARG);
    if (!prepare_kernels()) return record(QT_ERR_LAUNCH);
    const int sms = device_sm_count();
    const int tiles_m = (a.M + BM - 1) / BM;
    // Tile configuration.  The narrow tile with eight epilogue warps is the default: it holds a
    // thread's 64 partial sums without spilling and keeps twice the loads in flight for epilogues that
    // stream C, D and planes.  The wide tile needs 25 % less operand traffic per flop (the 128 x 128
    // tile is bound by operand delivery from L2) and is faster on a plain long-K product (280 vs
    // 289 us on 125 x 768^3), but its epilogue threads hold 128 partial sums and spill at the 168
    // registers a 320-thread CTA leaves them; over the whole optimizer step it loses 0.6 ms.  It
    // stays selectable (qt_gemm_force_tile) for measurements.
    int cfg = np == 3 ? 2 : 0;
    if (np == 2 && a.N > 128 && g_force_bn == 256) cfg = 1;
    // 128 x 192 tiles (eight epilogue warps of 96 columns, two operand stages, two accumulators): 17 % less
    // operand traffic per flop than 128 x 128 and, unlike 128 x 256, the 96 partial sums per thread
    // (nearly) fit the register budget.  Measured against 128 x 128: 125 x 768^3 371 -> 332 us,
    // 62 x 1200^3 868 -> 748, 36 x (768 x 3072 x 768) 489 -> 402, 8 x 4096^3 3653 -> 2882; with two
    // k-blocks only (1200 x 1200 x 128) it loses (169 -> 180), so short products stay on 128 x 128.
    // Products whose epilogue reads C and writes both fp32 and planes stay on 128 x 128 as well (the wide
    // epilogue is out of registers there: 600 x 1200 x 600 with all three 1.01 -> 1.10 ms per four launches).
    const bool heavy_epilogue = a.C && a.beta != 0.0f && a.D && a.Dhi;
    if (np == 2 && a.N > 128 && !qs && (g_force_bn == 192 || (g_force_bn == -1 && a.K >= 256 && !heavy_epilogue))) cfg = 5;
    if (qa || qb) cfg = 3;
    // CTA pairs (256-row bands) only on request: measured on B200 they are no faster than single
    // CTAs on 128 x 128 tiles (125 x 768^3: 372 vs 364 us; 8 x 4096^3: 3980 vs 3480 us) - halving
    // the B operand a CTA stages does not pay while each SM still multiplies 128 x 128 x 16 per
    // instruction; the 128 x 256 single-CTA tile is the one that gains (2900 us on the large case).
    const bool pair_possible = cfg == 0 && !qs && sms >= 2 && a.M > BM;
    if (pair_possible && g_force_bn == 512) cfg = 4;
    const bool pair = cfg == 4;
    const int bn = g_cfg_bn[cfg];
    GemmMaps maps;
    memset(&maps, 0, sizeof(maps));
    bool ok = true;
    for (int i = 0; i < 3; ++i) {
        const void *pa = Ap[i < np ? i : 0], *pb = Bp[i < np ? i : 0];
        const bool h = x.f16 != 0;
        if (qa) {}
        else if (!a.a_mn) ok = ok && make_map(&maps.a[i], pa, a.K, a.M, a_entries, a.lda, a.strideA, BK, BM, h);   // stored [M][K]
        else              ok = ok && make_map(&maps.a[i], pa, a.M, a.K, a_entries, a.lda, a.strideA, 64, BK, h);   // stored [K][M]
        if (qb) {}
        else if (!a.b_mn) ok = ok && make_map(&maps.b[i], pb, a.K, a.N, b_entries, a.ldb, a.strideB, BK, pair ? 64 : bn, h);   // stored [N][K]
        else              ok = ok && make_map(&maps.b[i], pb, a.N, a.K, b_entries, a.ldb, a.strideB, 64, BK, h);   // stored [K][N]
    }
    if (!ok) return record(QT_ERR_LAUNCH);
    GemmParams p;
    p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch; p.alpha = a.alpha; p.beta = a.beta;
    p.C = a.C; p.ldc = a.ldc; p.strideC = a.strideC; p.D = a.D; p.ldd = a.ldd; p.strideD = a.strideD;
    p.Dhi = static_cast<__nv_bfloat16 *>(a.Dhi); p.Dlo = static_cast<__nv_bfloat16 *>(a.Dlo);
    p.Dmid = static_cast<__nv_bfloat16 *>(x.Dmid);
    p.ldp = a.ldp; p.strideP = a.strideP;
    p.Thi = static_cast<__nv_bfloat16 *>(x.Thi); p.Tmid = static_cast<__nv_bfloat16 *>(x.Tmid); p.Tlo = static_cast<__nv_bfloat16 *>(x.Tlo);
    p.t_c0 = x.t_c0; p.t_c1 = x.t_c1; p.maxdev = x.maxdev;
    p.a_slot = x.a_slot; p.b_slot = x.b_slot; p.d_slot = x.d_slot; p.active = x.active;
    p.f16 = x.f16; p.a_exp = x.a_exp; p.b_exp = x.b_exp; p.ab_exp0 = x.ab_exp0;
    p.out_exp = x.out_exp; p.out_exp_w = x.out_exp_w; p.out_exp0 = x.out_exp0; p.out_rel = x.out_rel; p.kc = x.kc; p.c_follows_d = x.c_follows_d;
    p.aq = x.aq; p.bq = x.bq; p.oq_code = x.oq_code;
    p.tiles_m = pair ? (a.M + 2 * BM - 1) / (2 * BM) : tiles_m; p.tiles_n = (a.N + bn - 1) / bn;
    p.q_in = nullptr; p.q_absmax_in = p.q_diag_in = nullptr; p.q_out = nullptr; p.q_absmax_out = p.q_diag_out = nullptr;
    p.q_stride_codes = p.q_stride_absmax = p.q_stride_diag = 0; p.q_code = nullptr; p.q_nb = 0;
    if (qs) {
        p.q_in = qs->q_in; p.q_absmax_in = qs->absmax_in; p.q_diag_in = qs->q_in ? qs->diag_in : nullptr;
        p.q_out = qs->q_out; p.q_absmax_out = qs->absmax_out; p.q_diag_out = qs->diag_out;
        p.q_stride_codes = qs->stride_codes; p.q_stride_absmax = qs->stride_absmax; p.q_stride_diag = qs->stride_diag;
        p.q_code = qs->code; p.q_nb = (a.N + 63) / 64;
    }
    const long long ctas = (long long)p.tiles_m * p.tiles_n * a.batch;
    if (ctas > 0x7fffffffLL) return record(QT_ERR_UNSUPPORTED);
    GemmKern kern = g_kernels[cfg][a.a_mn ? 1 : 0][a.b_mn ? 1 : 0][qs ? 1 : 0];
    if (pair) {
        // persistent: one CTA pair (a cluster of two, scheduled on an SM pair) per two SMs
        long long pairs = ctas < sms / 2 ? ctas : sms / 2;
        if (x.max_ctas > 1 && pairs > x.max_ctas / 2) pairs = x.max_ctas / 2;
        cudaLaunchConfig_t cfgl;
        memset(&cfgl, 0, sizeof(cfgl));
        cfgl.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
        cfgl.blockDim = dim3((unsigned)g_cfg_threads[cfg], 1, 1);
        cfgl.dynamicSmemBytes = GEMM_SMEM;
        cfgl.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfgl.attrs = attr;
        cfgl.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfgl, kern, maps, p) != cudaSuccess) { cudaGetLastError(); return record(QT_ERR_LAUNCH); }
        count_launch(1);
        return check_launch();
    }
    unsigned grid = (unsigned)(ctas < sms ? ctas : sms);                         // persistent: one CTA per SM
    if (x.max_ctas > 0 && grid > (unsigned)x.max_ctas) grid = (unsigned)x.max_ctas;
    kern<<<grid, g_cfg_threads[cfg], GEMM_SMEM, s>>>(maps, p);
    count_launch(1);
    return check_launch();
}

// One product of the Newton chain: n x n, three planes in, three planes out (row-major
// operands: A is K-major, B is MN-major), with the optional extras of GemmExtras.
int launch_newton_product(void *const A[3], const int *a_slot, int a_entries,
                          void *const B[3], const int *b_slot, int b_entries,
                          void *const P[3], const int *d_slot, void *const T[3], float t_c0, float t_c1, float *maxdev,
                          const int *active, int n, int batch, long long ld, long long stride, cudaStream_t s) {
    GemmArgs a{A[0], A[2], ld, stride, 0, B[0], B[2], ld, stride, 1, n, n, n, batch, 1.0f, 0.0f,
               nullptr, 0, 0, nullptr, 0, 0, P[0], P[2], ld, stride};
    GemmExtras x;
    x.Dmid = P[1];
    x.Thi = T[0]; x.Tmid = T[1]; x.Tlo = T[2]; x.t_c0 = t_c0; x.t_c1 = t_c1;
    x.maxdev = maxdev; x.a_slot = a_slot; x.b_slot = b_slot; x.d_slot = d_slot; x.active = active;
    x.a_entries = a_entries; x.b_entries = b_entries;
    return launch_gemm_planes(a, A[1], B[1], s, nullptr, &x);
}

int launch_gemm_bf16x3(const GemmArgs &a, cudaStream_t s) { return launch_gemm_planes(a, nullptr, nullptr, s, nullptr); }

// fp32 operands in, fp32 out: both operands are split into bf16 planes inside `scratch`
// (global memory owned by the caller), then multiplied on the tensor cores.
static inline long long pitch8(long long cols) { return (cols + 7) / 8 * 8; }

// Bytes of plane scratch for one product; SIZE_MAX for negative or absurd sizes, so that a
// comparison against any real buffer size fails instead of wrapping around.
size_t matmul_f32_scratch_bytes(int M, int N, int K, int batch, int trans_a, int trans_b) {
    if (M < 0 || N < 0 || K < 0 || batch < 0) return SIZE_MAX;
    const unsigned __int128 a_rows = trans_a ? K : M, a_cols = trans_a ? M : K;
    const unsigned __int128 b_rows = trans_b ? N : K, b_cols = trans_b ? K : N;
    const unsigned __int128 elems = (unsigned __int128)batch * (a_rows * pitch8((long long)a_cols) + b_rows * pitch8((long long)b_cols));
    const unsigned __int128 bytes = elems * 2 /*planes*/ * 2 /*bytes*/ + 64;
    if (bytes > (unsigned __int128)1 << 46) return SIZE_MAX;             // 64 TiB: beyond any device
    return (size_t)bytes;
}

struct MatmulF32Args {
    const float *A; long long lda, strideA; int trans_a;
    const float *B; long long ldb, strideB; int trans_b;
    int M, N, K, batch; float alpha, beta;
    const float *C; long long ldc, strideC;
    float *D; long long ldd, strideD;
};

int launch_matmul_f32(const MatmulF32Args &a, void *scratch, size_t scratch_bytes, cudaStream_t s) {
    if (a.M < 0 || a.N < 0 || a.K <= 0 || a.batch < 0) return record(QT_ERR_ARG);
    if (a.M == 0 || a.N == 0 || a.batch == 0) return record(QT_OK);
    if (!a.A || !a.B || !a.D || !scratch) return record(QT_ERR_ARG);
    if (scratch_bytes < matmul_f32_scratch_bytes(a.M, a.N, a.K, a.batch, a.trans_a, a.trans_b)) return record(QT_ERR_ARG);
    const long long a_rows = a.trans_a ? a.K : a.M, a_cols = a.trans_a ? a.M : a.K;
    const long long b_rows = a.trans_b ? a.N : a.K, b_cols = a.trans_b ? a.K : a.N;
    const long long lpa = pitch8(a_cols), lpb = pitch8(b_cols);
    const long long spa = a_rows * lpa, spb = b_rows * lpb;              // plane strides per matrix
    unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(scratch) + 15) & ~(uintptr_t)15);
    __nv_bfloat16 *Ahi = reinterpret_cast<__nv_bfloat16 *>(base);
    __nv_bfloat16 *Alo = Ahi + (long long)a.batch * spa;
    __nv_bfloat16 *Bhi = Alo + (long long)a.batch * spa;
    __nv_bfloat16 *Blo = Bhi + (long long)a.batch * spb;
    int rc = launch_split_bf16(a.A, a.lda, a.strideA, (int)a_rows, (int)a_cols, a.batch, Ahi, Alo, lpa, spa, s);
    if (rc != QT_OK) return rc;
    rc = launch_split_bf16(a.B, a.ldb, a.strideB, (int)b_rows, (int)b_cols, a.batch, Bhi, Blo, lpb, spb, s);
    if (rc != QT_OK) return rc;
    // kernel convention: A logically M x K (a_mn: stored [K][M]); B logically N x K (b_mn: stored [K][N])
    GemmArgs g{Ahi, Alo, lpa, spa, a.trans_a ? 1 : 0, Bhi, Blo, lpb, spb, a.trans_b ? 0 : 1,
               a.M, a.N, a.K, a.batch, a.alpha, a.beta, a.C, a.ldc, a.strideC, a.D, a.ldd, a.strideD,
               nullptr, nullptr, 0, 0};
    return launch_gemm_bf16x3(g, s);
}

// ------------------------------------------------------------------------------------
// Allocation-free variant of launch_matmul_f32: the bf16 planes live in a fixed array that is
// part of the library image, so a caller that cannot obtain device memory at call time can
// still multiply fp32 matrices.  Every GPU that loads the library holds the array until the
// process exits.
// ------------------------------------------------------------------------------------
static constexpr size_t kStaticScratchBytes = (size_t)QT_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static void *g_static_scratch_addr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the CURRENT device.  In host code the array's name is
// only a handle; the address a kernel can use comes from cudaGetSymbolAddress, looked up once
// per device with that device current.
static int static_scratch_address(void **out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return QT_ERR_LAUNCH;
    if (!g_static_scratch_addr[dev]) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) {
            cudaGetLastError();
            return QT_ERR_LAUNCH;
        }
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return QT_OK;
}

int launch_matmul_f32_static(const MatmulF32Args &a, cudaStream_t s) {
    if (a.M < 0 || a.N < 0 || a.K <= 0 || a.batch < 0) return record(QT_ERR_ARG);
    if (a.M == 0 || a.N == 0 || a.batch == 0) return record(QT_OK);
    if (matmul_f32_scratch_bytes(a.M, a.N, a.K, a.batch, a.trans_a, a.trans_b) > kStaticScratchBytes)
        return record(QT_ERR_TOO_LARGE);
    void *scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != QT_OK) return record(rc);
    // Nothing in the scratch has to start at zero: the split kernels overwrite every plane
    // element the product reads (TMA never reads the pitch padding), so stale contents of an
    // earlier call are harmless.
    return launch_matmul_f32(a, scratch, kStaticScratchBytes, s);
}

// Self-test of the bounded waits: one CTA initialises an mbarrier that nothing ever arrives at
// and waits on it with the product kernel's own wait routine.  The wait must give up after
// WAIT_LIMIT polls, raise the CTA's abort flag and record QT_ERR_TIMEOUT in the device error
// word; the kernel then returns normally, so the context stays usable.
__global__ void k_selftest_wait_timeout(int *gave_up) {
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag);
        if (gave_up) *gave_up = ok ? 0 : 1;
    }
}

int launch_selftest_wait_timeout(int *gave_up_dev, cudaStream_t s) {
    k_selftest_wait_timeout<<<1, 32, 0, s>>>(gave_up_dev);
    count_launch(1);
    return check_launch();
}

int read_gemm_error(bool clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return QT_ERR_LAUNCH;
    if (clear && v != 0) {
        int z = 0;
        cudaMemcpyToSymbol(g_gemm_error, &z, sizeof(int));
    }
    return v;
}

}  // namespace qt

using namespace qt;

extern "C" {

int qt_split_bf16(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                  void *hi, void *lo, long long ldp, long long strideP, void *stream) {
    return launch_split_bf16(X, ldx, strideX, rows, cols, batch, hi, lo, ldp, strideP, static_cast<cudaStream_t>(stream));
}

int qt_split_bf16_rows(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                       const long long *index, long long stride_index, const float *scale, long long stride_scale,
                       void *hi, void *lo, long long ldp, long long strideP, void *stream) {
    return launch_split_bf16_rows(X, ldx, strideX, rows, cols, batch, index, stride_index, scale, stride_scale,
                                  hi, lo, ldp, strideP, static_cast<cudaStream_t>(stream));
}

int qt_gemm_bf16x3(const void *Ahi, const void *Alo, long long lda, long long strideA, int a_mn,
                   const void *Bhi, const void *Blo, long long ldb, long long strideB, int b_mn,
                   int M, int N, int K, int batch, float alpha, float beta,
                   const float *C, long long ldc, long long strideC,
                   float *D, long long ldd, long long strideD,
                   void *Dhi, void *Dlo, long long ldp, long long strideP, void *stream) {
    GemmArgs a{Ahi, Alo, lda, strideA, a_mn, Bhi, Blo, ldb, strideB, b_mn, M, N, K, batch, alpha, beta,
               C, ldc, strideC, D, ldd, strideD, Dhi, Dlo, ldp, strideP};
    return launch_gemm_bf16x3(a, static_cast<cudaStream_t>(stream));
}

int qt_split_bf16_3(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                    void *hi, void *mid, void *lo, long long ldp, long long strideP, void *stream) {
    return launch_split_bf16_3(X, ldx, strideX, rows, cols, batch, hi, mid, lo, ldp, strideP, static_cast<cudaStream_t>(stream));
}

int qt_gemm_bf16x6(const void *Ahi, const void *Amid, const void *Alo, long long lda, long long strideA, int a_mn,
                   const void *Bhi, const void *Bmid, const void *Blo, long long ldb, long long strideB, int b_mn,
                   int M, int N, int K, int batch, float alpha, float beta,
                   const float *C, long long ldc, long long strideC,
                   float *D, long long ldd, long long strideD, void *stream) {
    if (!Amid || !Bmid) return record(QT_ERR_ARG);
    GemmArgs a{Ahi, Alo, lda, strideA, a_mn, Bhi, Blo, ldb, strideB, b_mn, M, N, K, batch, alpha, beta,
               C, ldc, strideC, D, ldd, strideD, nullptr, nullptr, 0, 0};
    return launch_gemm_planes(a, Amid, Bmid, static_cast<cudaStream_t>(stream), nullptr);
}

int qt_gemm_bf16x3_q4(const void *Ahi, const void *Alo, long long lda, long long strideA, int a_mn,
                      const void *Bhi, const void *Blo, long long ldb, long long strideB, int b_mn,
                      int n, int K, int batch, float alpha, float beta, const float *code,
                      const unsigned char *q_in, const float *absmax_in, const float *diag_in,
                      unsigned char *q_out, float *absmax_out, float *diag_out,
                      long long stride_codes, long long stride_absmax, long long stride_diag, void *stream) {
    GemmArgs a{Ahi, Alo, lda, strideA, a_mn, Bhi, Blo, ldb, strideB, b_mn, n, n, K, batch, alpha, beta,
               nullptr, 0, 0, nullptr, 0, 0, nullptr, nullptr, 0, 0};
    QuantStateArgs qs{code, q_in, absmax_in, diag_in, q_out, absmax_out, diag_out, stride_codes, stride_absmax, stride_diag};
    return launch_gemm_planes(a, nullptr, nullptr, static_cast<cudaStream_t>(stream), &qs);
}

int qt_gemm_bf16x6_q4(const void *Ahi, const void *Amid, const void *Alo, long long lda, long long strideA, int a_mn,
                      const void *Bhi, const void *Bmid, const void *Blo, long long ldb, long long strideB, int b_mn,
                      int n, int K, int batch, float alpha, float beta, const float *code,
                      const unsigned char *q_in, const float *absmax_in, const float *diag_in,
                      unsigned char *q_out, float *absmax_out, float *diag_out,
                      long long stride_codes, long long stride_absmax, long long stride_diag, void *stream) {
    if (!Amid || !Bmid) return record(QT_ERR_ARG);
    GemmArgs a{Ahi, Alo, lda, strideA, a_mn, Bhi, Blo, ldb, strideB, b_mn, n, n, K, batch, alpha, beta,
               nullptr, 0, 0, nullptr, 0, 0, nullptr, nullptr, 0, 0};
    QuantStateArgs qs{code, q_in, absmax_in, diag_in, q_out, absmax_out, diag_out, stride_codes, stride_absmax, stride_diag};
    return launch_gemm_planes(a, Amid, Bmid, static_cast<cudaStream_t>(stream), &qs);
}

unsigned long long qt_matmul_f32_scratch_bytes(int M, int N, int K, int batch, int trans_a, int trans_b) {
    return (unsigned long long)matmul_f32_scratch_bytes(M, N, K, batch, trans_a, trans_b);
}

int qt_matmul_f32(const float *A, long long lda, long long strideA, int trans_a,
                  const float *B, long long ldb, long long strideB, int trans_b,
                  int M, int N, int K, int batch, float alpha, float beta,
                  const float *C, long long ldc, long long strideC,
                  float *D, long long ldd, long long strideD,
                  void *scratch, unsigned long long scratch_bytes, void *stream) {
    MatmulF32Args a{A, lda, strideA, trans_a, B, ldb, strideB, trans_b, M, N, K, batch, alpha, beta,
                    C, ldc, strideC, D, ldd, strideD};
    return launch_matmul_f32(a, scratch, (size_t)scratch_bytes, static_cast<cudaStream_t>(stream));
}

int qt_matmul_f32_static(const float *A, long long lda, long long strideA, int trans_a,
                         const float *B, long long ldb, long long strideB, int trans_b,
                         int M, int N, int K, int batch, float alpha, float beta,
                         const float *C, long long ldc, long long strideC,
                         float *D, long long ldd, long long strideD, void *stream) {
    MatmulF32Args a{A, lda, strideA, trans_a, B, ldb, strideB, trans_b, M, N, K, batch, alpha, beta,
                    C, ldc, strideC, D, ldd, strideD};
    return launch_matmul_f32_static(a, static_cast<cudaStream_t>(stream));
}

int qt_device_error(int clear) { return read_gemm_error(clear != 0); }

void qt_gemm_force_tile(int bn) { g_force_bn = bn; }

int qt_split_f16(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                 const long long *index, long long stride_index, const float *scale, long long stride_scale,
                 float *amax, int compute_amax, const int *exp_in, int target_or_exp0, int *exp_out,
                 void *hi, void *lo, long long ldp, long long strideP, void *stream) {
    return launch_split_f16(X, ldx, strideX, rows, cols, batch, index, stride_index, scale, stride_scale, amax, compute_amax, exp_in,
                            target_or_exp0, exp_out, hi, lo, ldp, strideP, static_cast<cudaStream_t>(stream));
}

int qt_gemm_ex(const qt_gemm_desc *d, void *stream) {
    if (!d) return record(QT_ERR_ARG);
    const bool three = d->A[1] != nullptr || d->B[1] != nullptr;
    GemmArgs a{d->A[0], d->A[2], d->lda, d->strideA, d->a_mn, d->B[0], d->B[2], d->ldb, d->strideB, d->b_mn,
               d->M, d->N, d->K, d->batch, d->alpha, d->beta, d->C, d->ldc, d->strideC, d->D, d->ldd, d->strideD,
               d->P[0], d->P[2], d->ldp, d->strideP};
    GemmExtras x;
    x.Dmid = d->P[1];
    x.Thi = d->T[0]; x.Tmid = d->T[1]; x.Tlo = d->T[2]; x.t_c0 = d->t_c0; x.t_c1 = d->t_c1;
    x.maxdev = d->maxdev; x.a_slot = d->a_slot; x.b_slot = d->b_slot; x.d_slot = d->d_slot; x.active = d->active;
    x.a_entries = d->a_entries; x.b_entries = d->b_entries;
    x.f16 = d->f16; x.a_exp = d->a_exp; x.b_exp = d->b_exp; x.ab_exp0 = d->ab_exp0;
    x.out_exp = d->out_exp; x.out_exp_w = d->out_exp_w; x.out_exp0 = d->out_exp0; x.out_rel = d->out_rel; x.kc = d->kc; x.max_ctas = d->max_ctas; x.c_follows_d = d->c_follows_d;
    if (d->aq_codes) x.aq = QOperand{d->aq_codes, d->aq_absmax, d->aq_diag, d->aq_slots, d->aq_stride_codes, d->aq_stride_absmax,
                                     d->aq_stride_diag, d->M, (d->M + 63) / 64};
    if (d->bq_codes) x.bq = QOperand{d->bq_codes, d->bq_absmax, d->bq_diag, d->bq_slots, d->bq_stride_codes, d->bq_stride_absmax,
                                     d->bq_stride_diag, d->N, (d->N + 63) / 64};
    x.oq_code = d->oq_code;
    if (three && (!d->A[1] || !d->B[1])) return record(QT_ERR_ARG);
    QuantStateArgs qs{d->q_code, d->q_in, d->q_absmax_in, d->q_diag_in, d->q_out, d->q_absmax_out, d->q_diag_out,
                      d->q_stride_codes, d->q_stride_absmax, d->q_stride_diag};
    return launch_gemm_planes(a, three ? d->A[1] : nullptr, three ? d->B[1] : nullptr, static_cast<cudaStream_t>(stream),
                              d->q_out ? &qs : nullptr, &x);
}

int qt_selftest_wait_timeout(int *gave_up, void *stream) {
    return launch_selftest_wait_timeout(gave_up, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
