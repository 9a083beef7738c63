/*
 * C ABI of libqtensor_b200.so: blockwise low-bit quantize / dequantize of square
 * preconditioner matrices and the dense products that run on that state, for
 * NVIDIA B200 (sm_100a).
 *
 * The first sixteen functions are a drop-in for the symbols that the reference's
 * ctypes loader binds (reference files: cudaC_python/csrc/pythonInterface.cpp:27-52,
 * bound in qtensor/functional.py:17-60 and called at :155, :211, :282, :343).  The
 * remaining qt_* functions are additive: status codes instead of exit(1), an explicit
 * CUDA stream, batched (strided) launches and the fused matrix kernels.
 *
 * Conventions (same as the reference, cudaC_python/csrc/ops.cu:4-174):
 *   - every pointer is a DEVICE pointer owned by the caller; the library keeps none
 *     after the call returns and never allocates or frees caller-visible memory;
 *   - matrices are square, order x order, row-major, contiguous;
 *   - absmax has order * ceil(order / blocksize) floats, indexed [row * nb + block];
 *   - packed output has ceil(order*order*bits/8) bytes;
 *   - launches are asynchronous on the calling thread's current stream
 *     (qt_set_stream; the legacy default stream until it is called).
 *
 * Byte format (that of the reference's CPU quantizer,
 * qtensor/functional.py:526-746): element 2j of the flat row-major index stream is the
 * HIGH nibble of byte j; an all-zero block stores code index 0 and dequantizes to +0.0;
 * normalisation is an IEEE fp32 division; ties between two codes go to the lower one.
 */
#ifndef QTENSOR_B200_H_
#define QTENSOR_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (qt_* functions return one; legacy void functions record it) ---- */
#define QT_OK                 0
#define QT_ERR_ARG            1   /* null pointer, negative size, misaligned buffer      */
#define QT_ERR_BLOCKSIZE      2   /* blocksize not in {64,128,256,512,1024,2048}         */
#define QT_ERR_BITS           3   /* bits not 4 or 8                                     */
#define QT_ERR_LAUNCH         4   /* CUDA reported an error at launch                    */
#define QT_ERR_DTYPE          5   /* dtype tag not QT_F32 / QT_BF16                      */
#define QT_ERR_UNSUPPORTED    6   /* shape outside what the kernel family supports       */
#define QT_ERR_TIMEOUT        7   /* a bounded device-side wait gave up                  */
#define QT_ERR_TOO_LARGE      8   /* operands exceed the fixed scratch of a *_static call */
#define QT_ERR_RANGE          9   /* a value left the range of a scaled fp16 operand plane */

/* Size of the built-in scratch array used by qt_matmul_f32_static (16 MiB per GPU). */
#define QT_STATIC_SCRATCH_BYTES (16u << 20)

#define QT_F32   0
#define QT_BF16  1

/* ---------------------------------------------------------------------------------- */
/* Legacy drop-in symbols.  Replace pythonInterface.cpp:29-51 one for one.            */
/* T* A is float* (fp32) or bf16 bits (bf16).  Return type is void as in the          */
/* reference; failures are recorded and readable through qt_last_error().             */
/* ---------------------------------------------------------------------------------- */
void cquantize_blockwise_8bit_bf16(void *A, float *code, int order, float *absmax, unsigned char *out, int blocksize);   /* pythonInterface.cpp:29 */
void cquantize_blockwise_8bit_fp32(float *A, float *code, int order, float *absmax, unsigned char *out, int blocksize);  /* :30 */
void cquantize_blockwise_4bit_bf16(void *A, float *code, int order, float *absmax, unsigned char *out, int blocksize);   /* :32 */
void cquantize_blockwise_4bit_fp32(float *A, float *code, int order, float *absmax, unsigned char *out, int blocksize);  /* :33 */
void cdequantize_blockwise_8bit_bf16(unsigned char *A, float *code, int order, float *absmax, void *out, int blocksize);  /* :35 */
void cdequantize_blockwise_8bit_fp32(unsigned char *A, float *code, int order, float *absmax, float *out, int blocksize); /* :36 */
void cdequantize_blockwise_4bit_bf16(unsigned char *A, float *code, int order, float *absmax, void *out, int blocksize);  /* :38 */
void cdequantize_blockwise_4bit_fp32(unsigned char *A, float *code, int order, float *absmax, float *out, int blocksize); /* :39 */
void cquantize_blockwise_diagreal_8bit_bf16(void *A, float *code, int order, float *absmax, float *diag, unsigned char *out, int blocksize);   /* :41 */
void cquantize_blockwise_diagreal_8bit_fp32(float *A, float *code, int order, float *absmax, float *diag, unsigned char *out, int blocksize);  /* :42 */
void cquantize_blockwise_diagreal_4bit_bf16(void *A, float *code, int order, float *absmax, float *diag, unsigned char *out, int blocksize);   /* :44 */
void cquantize_blockwise_diagreal_4bit_fp32(float *A, float *code, int order, float *absmax, float *diag, unsigned char *out, int blocksize);  /* :45 */
void cdequantize_blockwise_diagreal_8bit_bf16(unsigned char *A, float *code, int order, float *absmax, float *diag, void *out, int blocksize);  /* :47 */
void cdequantize_blockwise_diagreal_8bit_fp32(unsigned char *A, float *code, int order, float *absmax, float *diag, float *out, int blocksize); /* :48 */
void cdequantize_blockwise_diagreal_4bit_bf16(unsigned char *A, float *code, int order, float *absmax, float *diag, void *out, int blocksize);  /* :50 */
void cdequantize_blockwise_diagreal_4bit_fp32(unsigned char *A, float *code, int order, float *absmax, float *diag, float *out, int blocksize); /* :51 */

/* ---------------------------------------------------------------------------------- */
/* Additive entry points.                                                             */
/* ---------------------------------------------------------------------------------- */

/* Library ABI version (major*100 + minor). */
int qt_version(void);

/* Number of CUDA kernels this library has launched in this process (all threads).
 * Additive; the reference has no counterpart. */
unsigned long long qt_launch_count(void);

/* Accounting hook for callers that captured this library's launches in a CUDA graph: a replay
 * launches the captured kernels again without passing through the library, so the caller
 * reports how many of them one replay contained.  Additive; no counterpart in the reference. */
void qt_note_graph_replay(unsigned long long kernels);

/* Status of the most recent call made by this thread (legacy or qt_*), and its text.
 * Replaces the reference's fprintf + exit(1) (cudaC_python/csrc/ops.cuh:20-26). */
int qt_last_error(void);
const char *qt_error_string(int status);

/* Stream used by the legacy symbols on this thread (a cudaStream_t; NULL = legacy
 * default stream, which is what the reference always launches on, ops.cu:59). */
void qt_set_stream(void *stream);

/*
 * Batched strided quantize: `count` matrices of the same order, matrix m at
 * A + m*strideA elements, absmax + m*stride_absmax floats, diag + m*stride_diag floats
 * (diag == NULL selects the plain variant, otherwise the diagonal is kept in fp32 and
 * excluded from scale and codes), out + m*stride_out bytes.  One launch.
 * Follows quantizeBlockwise{4,8}bit[DiagReal] (ops.cu:4-64, :90-150) for each matrix.
 */
int qt_quantize_blockwise(const void *A, int a_dtype, long long strideA,
                          const float *code, int order, int count,
                          float *absmax, long long stride_absmax,
                          float *diag, long long stride_diag,
                          unsigned char *out, long long stride_out,
                          int blocksize, int bits, void *stream);

/* Batched strided dequantize; inverse of the above (ops.cu:66-88, :152-174). */
int qt_dequantize_blockwise(const unsigned char *A, long long strideA,
                            const float *code, int order, int count,
                            const float *absmax, long long stride_absmax,
                            const float *diag, long long stride_diag,
                            void *out, int out_dtype, long long stride_out,
                            int blocksize, int bits, void *stream);

/*
 * Dequantize into the operand format of the tcgen05 products (two bf16 planes hi, lo with
 * x = hi + lo to 16 bits, row pitch ldp elements, strideP elements between matrices; see
 * qt_split_bf16).  Output matrix j is read from state slot slots[j] (device int32 array), or
 * from slot j when slots is NULL; A, absmax and diag point at slot 0.  The values equal
 * qt_dequantize_blockwise followed by qt_split_bf16; the fp32 matrix, the gather of scattered
 * slots and the split pass never touch device memory.  This is the dequantize side of
 * preconditioned_grad (optimizers/shampoo2.py:258-268), where the dequantized preconditioners
 * are only ever product operands.  order must be a multiple of 8.
 */
int qt_dequantize_planes(const unsigned char *A, long long strideA, const float *code, int order, int count,
                         const float *absmax, long long stride_absmax, const float *diag, long long stride_diag,
                         const int *slots, void *hi, void *lo, long long ldp, long long strideP,
                         int blocksize, int bits, void *stream);

/*
 * qt_dequantize_planes into SCALED FP16 planes (operands of qt_gemm_ex with f16 != 0): entry =
 * value * 2^e[j], e[j] chosen from the largest magnitude matrix j can hold (its block scales and
 * fp32 diagonal) so that it lands just below 2^target; e is written to exp_out (count int32),
 * amax_scratch is `count` floats of device scratch.  22 significant bits instead of 16.
 */
int qt_dequantize_planes_f16(const unsigned char *A, long long strideA, const float *code, int order, int count,
                             const float *absmax, long long stride_absmax, const float *diag, long long stride_diag,
                             const int *slots, float *amax_scratch, int target, int *exp_out,
                             void *hi, void *lo, long long ldp, long long strideP, int blocksize, int bits, void *stream);

/*
 * Plane exponents of `count` matrices held as 4-bit state, without dequantizing them: e[j] puts
 * the largest magnitude matrix j (state slot slots[j], or j when slots is NULL) can hold - the
 * maximum over its block scales (n_absmax floats per slot) and, if diag is given, its fp32
 * diagonal (n_diag floats) - just below 2^target.  For qt_gemm_ex with aq_codes / bq_codes.
 */
int qt_state_exponents(const float *absmax, long long stride_absmax, int n_absmax,
                       const float *diag, long long stride_diag, int n_diag,
                       const int *slots, int count, int target, int *exp_out, void *stream);

/*
 * Self-test of the quantizer's division: the kernels replace x / absmax by an exact
 * reciprocal plus two fused corrections; this entry point compares that sequence with the
 * IEEE division on `pairs` pseudo-random operand pairs (seeded) and ADDS the number of
 * bitwise mismatches to *mismatches (device pointer, caller-initialised).  Expected: 0.
 * Additive; the reference divides directly (qtensor/functional.py:604).
 */
int qt_selftest_division(unsigned long long seed, unsigned long long pairs, unsigned long long *mismatches, void *stream);

/*
 * One 32-column panel step of a batched Householder QR (compact-WY form), the building
 * block that replaces the per-matrix torch.linalg.qr of the eigenbasis refresh
 * (reference: qtensor/utils.py:157).  For each of `count` row-major order x order
 * matrices (A + m*strideA floats) the columns j0 .. j0+width-1 (width <= 32), rows j0 ..
 * order-1, are factored.  Outputs, per matrix:
 *   V + m*strideV : order x order row-major; the block rows j0.., columns j0..j0+width-1
 *                   receives the Householder vectors (zeros above the diagonal, ones on it);
 *   T + m*strideT : 32 x 32 row-major upper-triangular factor with H_1..H_w = I - V T V^T.
 * A itself is only read.  Panels taller than 1216 rows are refused with QT_ERR_UNSUPPORTED
 * (the panel is held in registers, 38 rows per lane).
 */
int qt_householder_panel(const float *A, long long strideA, int order, int count, int j0, int width,
                         float *V, long long strideV, float *T, long long strideT, void *stream);

/*
 * qt_householder_panel preceded, in the same launch, by the rank-32 update the previous panel of
 * the same outer block leaves to do (right-looking blocked QR inside a block of up to four
 * panels ending at column block_end): with prev_width > 0 the block reflector of the panel at
 * columns j0-prev_width .. j0-1 (its vectors in V, its factor in Tprev + m*strideT) is applied
 * to columns j0 .. block_end-1, rows j0-prev_width .. order-1 of A IN PLACE (one CTA per matrix and
 * 32-column chunk), and the CTA of the first chunk then factors the panel at j0 as above.
 * prev_width == 0 is qt_householder_panel.  Replaces three library products per panel
 * (V^T C, T^T (.), C - V (.)) of a separately launched update.
 */
int qt_householder_panel_fused(float *A, long long strideA, int order, int count, int j0, int width,
                               float *V, long long strideV, float *T, long long strideT,
                               int prev_width, const float *Tprev, int block_end, void *stream);

/* Measurement / test hook: 0 (default) factors panels of more than 640 rows with the kernel that
 * gives a warp two columns (16 warps, the whole panel in registers) and shorter ones with one
 * column per warp (32 warps); 1 uses one column per warp at every height.  Additive. */
void qt_panel_force_form(int form);

/*
 * Triangular factor T (width x width, width <= 128) of a block of up to four consecutive panels,
 * H_1 .. H_width = I - Vo T Vo^T, from the panels' factors (Tp + m*strideTp: consecutive 32 x 32
 * row-major factors as written by qt_householder_panel) and the Gram matrix G = Vo^T Vo
 * (G + m*strideG, ldg floats between rows): LAPACK's larft recurrence on blocks.  T + m*strideT
 * is written whole, row-major, pitch `width`.  Part of the same replacement of
 * torch.linalg.qr (qtensor/utils.py:157).
 */
int qt_merge_t(const float *G, long long ldg, long long strideG, const float *Tp, long long strideTp, int width, int count,
               float *T, long long strideT, void *stream);

/*
 * fp32 matrix -> two bf16 planes, hi = bf16(x), lo = bf16(x - hi): the operand format of
 * qt_gemm_bf16x3.  X is rows x cols with ldx floats between rows, `batch` matrices strideX
 * floats apart; the planes have ldp elements between rows (a multiple of 8) and strideP
 * elements between matrices.  Additive; the reference multiplies fp32 tensors with
 * torch.matmul (e.g. optimizers/shampoo2.py:188-190).
 */
int qt_split_bf16(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                  void *hi, void *lo, long long ldp, long long strideP, void *stream);

/*
 * qt_split_bf16 with a row gather and / or a row scale: plane row i of matrix b holds
 * scale[b*stride_scale + i] * X[b][ index[b*stride_index + i] ][:] (index: int64 row numbers;
 * either pointer may be NULL).  Folds the selection of the kept eigenvector rows
 * (qtensor/utils.py:202, qtensor/functional.py:752) and the diag(.) factor of V^T diag(.) V
 * (qtensor/utils.py:203, qtensor/functional.py:762) into the operand preparation of the product.
 */
int qt_split_bf16_rows(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                       const long long *index, long long stride_index, const float *scale, long long stride_scale,
                       void *hi, void *lo, long long ldp, long long strideP, void *stream);

/*
 * Batched D = alpha * A * B^T-or-B + beta * C on the tcgen05 tensor cores with fp32
 * accumulation, operands as bf16 hi/lo planes (three MMAs per k-slice: hi*hi + hi*lo +
 * lo*hi, about 1e-5 relative accuracy).  Replaces the torch.matmul / @ products of the
 * reference's hot path (optimizers/shampoo2.py:188-199, :265-268; qtensor/utils.py:157-158,
 * :196, :203; qtensor/functional.py:757, :762; optimizers/matrix_functions.py:132-135).
 *   A is logically M x K: a_mn == 0 -> stored [M][K] (K contiguous), a_mn == 1 -> stored [K][M];
 *   B is logically N x K: b_mn == 0 -> stored [N][K],               b_mn == 1 -> stored [K][N];
 *   lda / ldb / strideA / strideB in bf16 elements, multiples of 8, bases 16-byte aligned;
 *   C (optional, fp32, ldc) and D (fp32, ldd) are row-major M x N; Dhi/Dlo (optional) receive
 *   D as bf16 planes (ldp).  At least one of D and Dhi/Dlo must be given.
 * Device-side waits are bounded; a wait that expires sets an error word readable with
 * qt_device_error() after synchronising.
 */
int qt_gemm_bf16x3(const void *Ahi, const void *Alo, long long lda, long long strideA, int a_mn,
                   const void *Bhi, const void *Blo, long long ldb, long long strideB, int b_mn,
                   int M, int N, int K, int batch, float alpha, float beta,
                   const float *C, long long ldc, long long strideC,
                   float *D, long long ldd, long long strideD,
                   void *Dhi, void *Dlo, long long ldp, long long strideP, void *stream);

/*
 * Three-plane variants (hi, mid, lo: x = hi + mid + lo to 24 bits; six MMAs per k-slice): the
 * same product at fp32-level accuracy (~1e-7 relative), for the two products of the hot path
 * whose result must resolve eigenvalues down to 1e-7 of the largest one
 * (beta L + (1-beta) G G^T, optimizers/shampoo2.py:188-199, and L V of the Rayleigh quotients,
 * qtensor/utils.py:158).  Arguments as qt_split_bf16 / qt_gemm_bf16x3 with one more plane;
 * only an fp32 D is produced.
 */
int qt_split_bf16_3(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                    void *hi, void *mid, void *lo, long long ldp, long long strideP, void *stream);
int qt_gemm_bf16x6(const void *Ahi, const void *Amid, const void *Alo, long long lda, long long strideA, int a_mn,
                   const void *Bhi, const void *Bmid, const void *Blo, long long ldb, long long strideB, int b_mn,
                   int M, int N, int K, int batch, float alpha, float beta,
                   const float *C, long long ldc, long long strideC,
                   float *D, long long ldd, long long strideD, void *stream);

/*
 * General form of the two products above, for chains of products that hand bf16 planes from one
 * epilogue to the next prologue (the coupled Newton iteration of the inverse root,
 * optimizers/matrix_functions.py:127-140: root * T, T^2, T^4, T^4 * M, max |M - I|):
 *   - A, B: planes {hi, mid, lo}; mid == NULL on both selects the two-plane product (three MMAs),
 *     otherwise the three-plane one (six MMAs);
 *   - result as fp32 D and / or as planes P {hi, mid, lo} (mid only for three-plane products);
 *   - T (three-plane products): also writes t_c0 * I + t_c1 * result as three planes, same pitch;
 *   - maxdev: per matrix, max |result - I| is combined into maxdev[m] with an atomic maximum
 *     (non-negative floats; the caller zeroes it; NaN / inf count as +inf);
 *   - a_slot / b_slot / d_slot: per matrix, which entry of A's / B's storage is read and which
 *     entry of the outputs is written (NULL: the matrix number); a_entries / b_entries give the
 *     number of matrices in A's / B's storage (0: batch);
 *   - active: per matrix, 0 = skip all tiles of this matrix (NULL: none skipped);
 *   - f16 != 0 (two-plane products): the planes are SCALED FP16 planes - an entry holds
 *     value * 2^(exp[entry] + exp0) as hi = fp16(.), lo = fp16(. - hi), 22 significant bits while
 *     the scaled values stay within fp16's normal range (qt_planes_exponents picks exponents from
 *     each matrix's largest magnitude).  a_exp / b_exp: per storage entry exponents (NULL: 0),
 *     ab_exp0: sum of the two common parts; the epilogue undoes the scaling.  Plane output P
 *     then is fp16 too, entry = value * 2^e with e = out_exp[entry] + out_exp0 if out_exp is
 *     given, else (out_rel != 0) the operands' exponents + out_exp0, else out_exp0; e is written
 *     to out_exp_w[entry] if that is given.  A value that leaves the fp16 range is clamped and
 *     sets the sticky device error QT_ERR_RANGE.  kc: k-blocks (of 64) per accumulation chain in
 *     tensor memory, partial sums added in fp32 registers (0: one chain; the tensor core's
 *     accumulation truncates, so long chains lose about 6.5e-9 * K);
 *   - q_out != NULL: the result is written as 4-bit state exactly as qt_gemm_bf16x3_q4 does
 *     (q_* fields as that function's arguments), instead of D / P;
 *   - aq_codes / bq_codes != NULL (f16 products with row-major operands: a_mn == 0, b_mn == 1):
 *     that operand is not read from planes but DEQUANTIZED INSIDE THE KERNEL from 4-bit block-64
 *     state (square, order M for A and N for B, K equal to it): converter warps turn each
 *     128-byte line of the operand tile from codes and block scales (diagonal from *_diag, may be
 *     NULL) into the swizzled fp16 hi / lo tile the tensor core reads, so neither the fp32
 *     matrix nor its operand planes exist in device memory.  Matrix m of the product is state
 *     slot *_slots[m] (NULL: m) of storage laid out with the *_stride_* strides (bytes / floats /
 *     floats per slot); its plane exponent is a_exp[m] / b_exp[m] (see qt_state_exponents);
 *     oq_code is the 16-entry codebook.  The tile bytes equal those qt_dequantize_planes_f16
 *     writes.  This is the operand side of preconditioned_grad (optimizers/shampoo2.py:255-268).
 * All index, exponent and flag arrays are device int32 arrays read when the kernel runs.
 */
typedef struct qt_gemm_desc {
    const void *A[3]; long long lda, strideA; int a_mn, a_entries;
    const void *B[3]; long long ldb, strideB; int b_mn, b_entries;
    int M, N, K, batch; float alpha, beta;
    const float *C; long long ldc, strideC;
    float *D; long long ldd, strideD;
    void *P[3]; long long ldp, strideP;
    void *T[3]; float t_c0, t_c1;
    float *maxdev;
    const int *a_slot, *b_slot, *d_slot, *active;
    int f16, ab_exp0, out_exp0, out_rel, kc;
    const int *a_exp, *b_exp, *out_exp; int *out_exp_w;
    const float *q_code; const unsigned char *q_in; const float *q_absmax_in, *q_diag_in;
    unsigned char *q_out; float *q_absmax_out, *q_diag_out;
    long long q_stride_codes, q_stride_absmax, q_stride_diag;
    const float *oq_code;
    const unsigned char *aq_codes; const float *aq_absmax, *aq_diag; const int *aq_slots;
    long long aq_stride_codes, aq_stride_absmax, aq_stride_diag;
    const unsigned char *bq_codes; const float *bq_absmax, *bq_diag; const int *bq_slots;
    long long bq_stride_codes, bq_stride_absmax, bq_stride_diag;
    int max_ctas;   /* > 0: at most this many CTAs (the kernel is persistent and otherwise takes every SM until
                     * it is done, so a latency-critical kernel launched beside it on another stream would wait for
                     * the whole product); 0: one CTA per SM */
    int c_follows_d; /* != 0: the C operand of matrix b is entry d_slot[b] of its array, like the outputs
                      * (C == D then updates selected entries of an array in place) */
} qt_gemm_desc;
int qt_gemm_ex(const qt_gemm_desc *desc, void *stream);

/*
 * Largest eigenvalue of each of `batch` symmetric n x n fp32 matrices (G + m*strideG) by power
 * iteration from the given start vectors v0 (batch x n), following PowerIter of the reference
 * (optimizers/matrix_functions.py:22-48) step by step: normalise, multiply, Rayleigh quotient,
 * stop when the quotient moves by <= tol or after max_iters steps.  One launch for the batch, no
 * host synchronisation (the reference synchronises once per step, :40).  max_ev: batch floats;
 * iters (may be NULL): steps taken per matrix; vec (may be NULL): batch x n, the last iterate G v
 * (not normalised).
 */
int qt_power_iter(float *G, long long strideG, int n, int batch, const float *v0, float tol, int max_iters,
                  float *max_ev, int *iters, float *vec, void *stream);

/*
 * (G + ridge_eps * lambda_max(G) I)^(-1/p) for `batch` SPD fp32 matrices by the coupled Newton
 * iteration, i.e. ComputePower of the reference (optimizers/matrix_functions.py:80-141; callers
 * optimizers/shampoo1.py:181-201 and optimizers/shampoo2.py:220-230) for a whole batch:
 * power iteration from v0 (batch x n; the reference draws torch.rand(n) * 2 - 1 per matrix),
 * ridge added to G's diagonal IN PLACE (as the reference does, :112), then up to iter_count
 * iterations root' = root T, M' = T^p M with every product on the three-plane tcgen05 kernel,
 * max |M' - I| reduced in the epilogue and the reference's accept / stop rule (:131-140) applied
 * per matrix through flags in device memory - no host synchronisation anywhere.
 * p must be a power of two >= 2 (the optimizers use 4).  workspace: caller-owned device memory of
 * qt_inverse_root_newton_workspace_bytes(n, batch) bytes, 256-byte aligned (42 bytes per matrix
 * element: ping-pong planes of M and root, T and two powers of T).  out + m*strideOut: n x n fp32.
 * max_ev, iters (may be NULL): per matrix lambda_max estimate and accepted iterations.
 */
unsigned long long qt_inverse_root_newton_workspace_bytes(int n, int batch);
int qt_inverse_root_newton(float *G, long long strideG, int n, int batch, int p, int iter_count, float tol, float ridge_eps,
                           const float *v0, void *workspace, unsigned long long workspace_bytes,
                           float *out, long long strideOut, float *max_ev, int *iters, void *stream);

/*
 * fp32 matrices -> scaled fp16 planes (the operand format of qt_gemm_ex with f16 != 0), with the
 * optional row gather and row scale of qt_split_bf16_rows.  Plane entry = x * 2^e[b] as
 * hi = fp16(.), lo = fp16(. - hi).  Exponents:
 *   amax != NULL: e[b] is chosen from amax[b] so that a magnitude of amax[b] lands just below
 *     2^target_or_exp0.  compute_amax != 0: amax is `batch` floats of scratch and is filled here
 *     with each matrix's largest magnitude (one extra pass over X); compute_amax == 0: amax holds
 *     upper bounds the caller already knows (a value above its bound is clamped in the planes);
 *   amax == NULL: e[b] = exp_in[b] (NULL: 0) + target_or_exp0.
 * exp_out (may be NULL) receives e[b].  Additive; the reference multiplies fp32 tensors with
 * torch.matmul (e.g. optimizers/shampoo2.py:188-190).
 */
int qt_split_f16(const float *X, long long ldx, long long strideX, int rows, int cols, int batch,
                 const long long *index, long long stride_index, const float *scale, long long stride_scale,
                 float *amax, int compute_amax, const int *exp_in, int target_or_exp0, int *exp_out,
                 void *hi, void *lo, long long ldp, long long strideP, void *stream);

/* Measurement / test hook for the tile configuration of two-plane products.  -1 (default): 128 x 192
 * tiles for plain products wider than 128 columns with K >= 256, else 128 x 128; 128, 192, 256: single
 * CTAs with that tile width wherever the variant exists; 512: CTA pairs (tcgen05 cta_group::2: two CTAs
 * of a cluster on one 256 x 128 tile, each staging its rows of A and half of B) wherever they are
 * possible (plain epilogue, more than 128 rows).  All of them give the same bits.  Additive; no
 * counterpart in the reference. */
void qt_gemm_force_tile(int bn);

/*
 * The three-product (qt_gemm_bf16x3_q4) and six-product (qt_gemm_bf16x6_q4) GEMMs with 4-bit
 * blockwise state (block size 64, the byte format of qt_quantize_blockwise) as C operand and as
 * result, square n x n, n a multiple of 16:
 *     state_out = quantize( alpha * op(A) * op(B) + beta * dequantize(state_in) )
 * The old state is dequantized and the new one quantized inside the epilogue, so no fp32 copy of
 * the state is written to or read from device memory; the bytes equal those of
 * qt_dequantize_blockwise -> qt_gemm_bf16x3 / x6 -> qt_quantize_blockwise.  This is the fused form of
 * the statistics update L <- beta L + (1-beta) G G^T (optimizers/shampoo1.py:163-179: product,
 * dequantize, mul_/add_, quantize) and of storing a product as a low-bit preconditioner
 * (optimizers/shampoo2.py:231).
 * q_in == NULL: no C operand (beta ignored).  diag_out != NULL selects the diagreal variant for
 * the result, diag_in != NULL for the operand.  q_out may equal q_in (update in place).
 * Strides are per matrix: stride_codes in bytes (a multiple of 8), stride_absmax and stride_diag
 * in floats; code pointers must be 8-byte aligned.
 */
int qt_gemm_bf16x3_q4(const void *Ahi, const void *Alo, long long lda, long long strideA, int a_mn,
                      const void *Bhi, const void *Blo, long long ldb, long long strideB, int b_mn,
                      int n, int K, int batch, float alpha, float beta, const float *code,
                      const unsigned char *q_in, const float *absmax_in, const float *diag_in,
                      unsigned char *q_out, float *absmax_out, float *diag_out,
                      long long stride_codes, long long stride_absmax, long long stride_diag, void *stream);
int qt_gemm_bf16x6_q4(const void *Ahi, const void *Amid, const void *Alo, long long lda, long long strideA, int a_mn,
                      const void *Bhi, const void *Bmid, const void *Blo, long long ldb, long long strideB, int b_mn,
                      int n, int K, int batch, float alpha, float beta, const float *code,
                      const unsigned char *q_in, const float *absmax_in, const float *diag_in,
                      unsigned char *q_out, float *absmax_out, float *diag_out,
                      long long stride_codes, long long stride_absmax, long long stride_diag, void *stream);

/*
 * D = alpha * op(A) * op(B) + beta * C for fp32 row-major operands in one call: splits both
 * operands into bf16 planes inside `scratch` (caller-owned device memory of at least
 * qt_matmul_f32_scratch_bytes(...) bytes), then runs qt_gemm_bf16x3.  op(A) is M x K
 * (trans_a: A is stored K x M), op(B) is K x N (trans_b: B is stored N x K); lda/ldb/ldc/ldd in
 * floats, `batch` matrices stride* floats apart.  Same products of the reference as
 * qt_gemm_bf16x3 (e.g. qtensor/utils.py:196, optimizers/shampoo2.py:265-268).
 */
unsigned long long qt_matmul_f32_scratch_bytes(int M, int N, int K, int batch, int trans_a, int trans_b);
int qt_matmul_f32(const float *A, long long lda, long long strideA, int trans_a,
                  const float *B, long long ldb, long long strideB, int trans_b,
                  int M, int N, int K, int batch, float alpha, float beta,
                  const float *C, long long ldc, long long strideC,
                  float *D, long long ldd, long long strideD,
                  void *scratch, unsigned long long scratch_bytes, void *stream);

/*
 * qt_matmul_f32 for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Who needs it: a host that gave its whole device-memory budget to a fixed arena
 * at start-up and has no allocator to ask at call time; a plain-C embedding with no tensor
 * library behind it; a latency-critical loop where an allocation (which may synchronise the
 * device or fail under fragmentation) is not acceptable.  Such callers still own A, B, C and D;
 * what they cannot supply is the temporary room for the bf16 operand planes.  This entry point
 * keeps that room inside the library: a fixed QT_STATIC_SCRATCH_BYTES (16 MiB) array in device
 * memory, present on every GPU that loads the library for the life of the process.
 *   - Arguments and result are those of qt_matmul_f32 without `scratch`; the output is
 *     bit-identical to qt_matmul_f32 on the same inputs.
 *   - Limit: qt_matmul_f32_scratch_bytes(M, N, K, batch, trans_a, trans_b) must not exceed
 *     QT_STATIC_SCRATCH_BYTES (e.g. two 1024 x 1024 operands, or 16 pairs of 256 x 256);
 *     larger requests return QT_ERR_TOO_LARGE and launch nothing.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress with that device current).  Make that first call during set-up,
 *     before any stream capture is begun on that device.
 *   - All calls on one GPU share the one array, which keeps whatever the previous call left in
 *     it; nothing in it needs to be cleared between calls.  Two calls whose kernels can overlap
 *     on the GPU (different streams, no ordering between them) race on the array: order them.
 */
int qt_matmul_f32_static(const float *A, long long lda, long long strideA, int trans_a,
                         const float *B, long long ldb, long long strideB, int trans_b,
                         int M, int N, int K, int batch, float alpha, float beta,
                         const float *C, long long ldc, long long strideC,
                         float *D, long long ldd, long long strideD, void *stream);

/*
 * Fused AdamW tail of the Shampoo step over a list of fp32 tensors, one launch
 * (optimizers/shampoo2.py:441 and :457-466: decoupled weight decay, both moments, bias-corrected
 * update), d being the preconditioned and grafted direction:
 *     p <- p * scalars[2];  m <- beta1 m + (1-beta1) d;  v <- beta2 v + (1-beta2) d d;
 *     p <- p + scalars[1] * m / (sqrt(v) * scalars[0] + eps)
 * with scalars = { 1/sqrt(1-beta2^t), -lr/(1-beta1^t), 1 - lr*weight_decay } in DEVICE memory.
 * one_minus_beta{1,2} are passed separately because the reference forms 1 - beta in double
 * precision before rounding (1 - 0.999 differs from 1.0f - 0.999f by 1.3e-5 relative).
 * All tables are device arrays: per tensor the four addresses (as 64-bit integers) and the
 * element count; per CTA a (tensor, chunk) pair; a chunk is chunk_elems elements (a multiple of 4).
 */
int qt_adamw_tail(const long long *p_ptrs, const long long *d_ptrs, const long long *m_ptrs, const long long *v_ptrs,
                  const long long *numels, const int *chunk_tensor, const int *chunk_index, int num_chunks,
                  int chunk_elems, const float *scalars, float beta1, float beta2, float one_minus_beta1,
                  float one_minus_beta2, float eps, void *stream);

/*
 * out[b][j] = sum_i A[b][i][j] * B[b][i][j] for `batch` pairs of row-major fp32 matrices (rows x cols,
 * row pitch ld, matrix stride `stride`, both operands alike): the Rayleigh quotients diag(V^T L V) of
 * the eigenbasis refresh (qtensor/utils.py:158) from L V and V.  The order of summation depends on
 * rows and cols only, never on the batch.  Additive.
 */
int qt_column_dot(const float *A, const float *B, long long ld, long long stride, int rows, int cols, int batch,
                  float *out, long long stride_out, void *stream);

/* Sticky device-side error word (QT_OK or QT_ERR_TIMEOUT); synchronises the device.
 * clear != 0 resets it.  Additive; the reference has no device-side waits. */
int qt_device_error(int clear);

/*
 * Self-test of the bounded device-side waits: launches one CTA that waits, with the product
 * kernels' own wait routine, on an mbarrier that nothing arrives at.  The wait gives up after
 * its poll limit (well under a second), writes 1 to *gave_up (device int, may be NULL) and sets
 * the sticky error word to QT_ERR_TIMEOUT; the kernel returns normally and the context stays
 * usable.  Additive; the reference has no device-side waits (its only failure path is
 * exit(1), cudaC_python/csrc/ops.cuh:20-26).
 */
int qt_selftest_wait_timeout(int *gave_up, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* QTENSOR_B200_H_ */
