/* C ABI of the B200 prover core (libzkllm_b200.so).
 *
 * The reference implementation has no FFI layer: its operator surface is the set
 * of C++ classes in its .cuh headers.  Each entry point below replaces the device
 * work behind one of those methods; the comment in front of it names the method
 * (file:line within the reference project).  The C++ classes of the same names
 * in zkllm-ccs2024_b200/host/ forward to these calls.
 *
 * Conventions
 *  - Every function returns ZKB_OK (0) or a negative ZKB_ERR_* code;
 *    zkb_last_error() gives the text for the calling thread.  No exception
 *    crosses this boundary.
 *  - Pointers named d_* are device addresses, h_* are host addresses.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *    stream).  Calls that return values through h_* pointers synchronise the
 *    stream before returning; all others are asynchronous on `stream`.
 *  - Fr elements are 8 little-endian u32 limbs in STANDARD (non-Montgomery)
 *    form, canonical in [0, r), 32 bytes, 16-byte aligned — the reference's
 *    Fr_t / FrTensor layout (bls12-381.cuh:116-120).
 *  - G1 points are Jacobian (X, Y, Z) triples of 12-limb Fq values in MONTGOMERY
 *    form, 144 bytes; Z == 0 is the identity — the reference's G1Jacobian_t /
 *    G1TensorJacobian layout (bls12-381.cuh:429-433).  Affine points are 96
 *    bytes (X, Y).
 *  - Challenge vectors are host arrays of Fr in standard form, in the order the
 *    reference's functions take them.
 */
#ifndef ZKLLM_B200_H
#define ZKLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZKB_OK            0
#define ZKB_ERR_CUDA     (-1)  /* a CUDA call failed                                   */
#define ZKB_ERR_DIM      (-2)  /* incompatible dimensions (reference: runtime_error)   */
#define ZKB_ERR_VERIFY   (-3)  /* a verifier equation failed (reference: runtime_error) */
#define ZKB_ERR_ARG      (-4)  /* invalid argument                                     */
#define ZKB_ERR_LIMIT    (-5)  /* size beyond a documented limit                       */

typedef struct { uint32_t val[8]; }  zkb_fr_t;        /* Fr_t          */
typedef struct { uint32_t val[12]; } zkb_fq_t;        /* Fp_t          */
typedef struct { zkb_fq_t x, y; }    zkb_g1_affine_t; /* G1Affine_t    */
typedef struct { zkb_fq_t x, y, z; } zkb_g1_t;        /* G1Jacobian_t  */

/* ---- library ---------------------------------------------------------------- */
const char* zkb_last_error(void);
int zkb_version(void);
/* Number of kernels this library has launched in the calling process. */
unsigned long long zkb_launch_count(void);

/* Per-kernel timing for benchmarks (no counterpart in the reference).  While
 * enabled, every kernel launch of the library is bracketed by CUDA events on its
 * stream.  zkb_profile_read synchronises the device and writes one line per
 * kernel, "name,launches,total_ms\n", into buf, followed by "host:<call>,calls,total_ms"
 * lines for the host time spent in the device-memory allocator. */
int zkb_profile_enable(int on);
int zkb_profile_reset(void);
int zkb_profile_read(char* buf, size_t cap);

/* Integer-pipe micro-benchmark (no counterpart in the reference): issue rate, in
 * 10^9 instructions per second, of mode 0 = mad.lo.u32, 1 = mad.wide.u32,
 * 2 = the mad.lo.cc/madc.hi.cc carry chains of the field multiplier. */
int zkb_bench_imad(int mode, unsigned iters, double* h_gops, void* stream);

/* ---- device memory (FrTensor/G1Tensor ctors, dtors, copies:
 *      fr-tensor.cu:158-179, g1-tensor.cu:40-60,123-152) ------------------------- */
int zkb_malloc(void** d_ptr, size_t bytes);   /* usable at once on any stream */
int zkb_free(void* d_ptr);                     /* waits for the device first, like cudaFree */
/* zkb_free for a buffer that only the default stream (and the library's calls on it) has used: waits for the
 * default stream instead of the whole device, so openings in flight (zkb_me_open_begin) keep running. */
int zkb_free_default_stream(void* d_ptr);
/* Device memory of this library (zkb_malloc and the scratch memory of every call) comes from a
 * stream-ordered pool the library owns, which keeps freed blocks for reuse (no counterpart in the reference,
 * which calls cudaMalloc / cudaFree per tensor, fr-tensor.cu:158-179).  zkb_pool_trim waits for the device and
 * returns cached memory to the driver down to keep_bytes. */
int zkb_pool_trim(size_t keep_bytes);
/* Streams (no counterpart in the reference, which works on the default stream only).  zkb_stream_create makes a
 * non-blocking stream of the highest (or lowest) priority the device offers.  zkb_set_default_stream names the stream
 * that a null `stream` argument stands for from then on, in every entry point and in zkb_malloc / zkb_free_default_stream
 * (null again: the CUDA default stream).  A host that starts openings with zkb_me_open_begin and keeps proving can give
 * its own work a high-priority stream this way: its short kernels are then scheduled ahead of the openings' long blocks.
 * The setting is process-wide; change it only while nothing is in flight. */
int zkb_stream_create(int high_priority, void** stream);
int zkb_stream_destroy(void* stream);
int zkb_set_default_stream(void* stream);
/* Guard bands around every block the library hands out (debug aid, no counterpart in the reference; also switched on
 * by ZKLLM_GUARD=1 in the environment): 256 bytes of a fixed pattern before and after each scratch block and each
 * zkb_malloc buffer allocated while it is on, compared with the pattern when the block is released.
 * zkb_guard_report waits for the device and returns how many blocks were checked, how many had a band written, the
 * size in bytes of the first such block and its side (0 = before, 1 = after, -1 = none); reset != 0 clears the counts. */
int zkb_guard_enable(int on);
int zkb_guard_report(unsigned long long* blocks_checked, unsigned long long* blocks_damaged,
                     unsigned long long* first_damaged_bytes, int* first_damaged_side, int reset);
/* Page-locked host memory and copies that do not wait (no counterpart in the
 * reference, whose ioutils.cu:3-45 stages files through pageable memory): the host
 * buffer must stay untouched until zkb_sync on the same stream. */
int zkb_host_alloc(void** h_ptr, size_t bytes);
int zkb_host_free(void* h_ptr);
int zkb_memcpy_h2d_async(void* d_dst, const void* h_src, size_t bytes, void* stream);
int zkb_memcpy_d2h_async(void* h_dst, const void* d_src, size_t bytes, void* stream);
int zkb_memcpy_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream);
int zkb_memcpy_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream);
int zkb_memcpy_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream);
int zkb_memset0(void* d_dst, size_t bytes, void* stream);
int zkb_sync(void* stream);

/* ---- fixed-point <-> Fr (fr-tensor.cu:186-236, 713-798) ------------------------ */
int zkb_fr_from_i32(const int32_t* d_in, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_from_i64(const int64_t* d_in, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_to_i32(const zkb_fr_t* d_in, int32_t* d_out, size_t n, void* stream);
int zkb_fr_to_i64(const zkb_fr_t* d_in, int64_t* d_out, size_t n, void* stream);
int zkb_fr_from_f32(const float* d_in, uint64_t scale, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_from_f64(const double* d_in, uint64_t scale, zkb_fr_t* d_out, size_t n, void* stream);

/* ---- elementwise field ops (FrTensor operators, fr-tensor.cu:257-373).
 *      d_out may alias an input.  The *_scalar forms broadcast one host value. ---- */
int zkb_fr_add(const zkb_fr_t* d_a, const zkb_fr_t* d_b, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_sub(const zkb_fr_t* d_a, const zkb_fr_t* d_b, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_mul(const zkb_fr_t* d_a, const zkb_fr_t* d_b, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_neg(const zkb_fr_t* d_a, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_add_scalar(const zkb_fr_t* d_a, const zkb_fr_t* h_x, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_sub_scalar(const zkb_fr_t* d_a, const zkb_fr_t* h_x, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_mul_scalar(const zkb_fr_t* d_a, const zkb_fr_t* h_x, zkb_fr_t* d_out, size_t n, void* stream);
/* FrTensor::mont / unmont (fr-tensor.cu:323-337): multiply by 2^256 / 2^-256 mod r */
int zkb_fr_mont(const zkb_fr_t* d_a, zkb_fr_t* d_out, size_t n, void* stream);
int zkb_fr_unmont(const zkb_fr_t* d_a, zkb_fr_t* d_out, size_t n, void* stream);
/* Fr_elementwise_mont_mul (fr-tensor.cu:126): a*b*2^-256 mod r */
int zkb_fr_mont_mul(const zkb_fr_t* d_a, const zkb_fr_t* d_b, zkb_fr_t* d_out, size_t n, void* stream);
/* 1/(a + beta), zero mapped to zero (tlookup_inv_kernel, tlookup.cu:50-62) */
int zkb_fr_inv_shifted(const zkb_fr_t* d_a, const zkb_fr_t* h_beta, zkb_fr_t* d_out, size_t n, void* stream);

/* ---- reductions and multilinear folds ------------------------------------------ */
/* FrTensor::sum (fr-tensor.cu:406-434) */
int zkb_fr_sum(const zkb_fr_t* d_a, size_t n, zkb_fr_t* h_out, void* stream);
/* FrTensor::operator()(u) (fr-tensor.cu:437-442): multilinear extension at u, u[0]
 * binding the least-significant index bit; needs 2^(k-1) < n <= 2^k. */
int zkb_fr_mle_eval(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k,
                    zkb_fr_t* h_out, void* stream);
/* Same evaluation for callers that cannot allocate device memory - for example a
 * process that gave the whole GPU to its own memory manager at start-up, or a
 * latency-critical loop that must stay clear of the allocator.  It has no
 * counterpart in the reference.  All working memory is one fixed device array
 * inside the library (288 KiB on every GPU that loads the library, held until
 * exit); the call performs no cudaMalloc/cudaFree and uses no memory pool.
 * Limit: n <= 2^24 elements (k <= 24), larger sizes return ZKB_ERR_LIMIT.
 * The first call on a device looks up the array's address; make that first
 * call before any stream capture.  All calls share the array, so two calls
 * that overlap on the GPU (different streams or threads) race: serialise them. */
int zkb_fr_mle_eval_noalloc(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k,
                            zkb_fr_t* h_out, void* stream);
/* FrTensor::partial_me(u, cur_dim, window_size) (fr-tensor.cu:518-560): the tensor
 * is [n/(cur_dim*window), cur_dim, window]; the middle axis is folded away with u.
 * d_out receives n/cur_dim elements. */
int zkb_fr_partial_me(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k,
                      size_t cur_dim, size_t window, zkb_fr_t* d_out, void* stream);
/* FrTensor::partial_me(u, window_size) (fr-tensor.cu:512-516, 612-641): folds
 * consecutive windows pairwise k times; d_out receives
 * window * ceil(ceil(n/window) / 2^k) elements (*out_n is set to that count). */
int zkb_fr_partial_me_window(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k,
                             size_t window, zkb_fr_t* d_out, size_t* out_n, void* stream);
/* FrTensor::multi_dim_me (fr-tensor.cu:643-652) for a [d0, d1] tensor:
 * folds axis 1 with u1 (k1 values) and then axis 0 with u0 (k0 values). */
int zkb_fr_mle_eval_2d(const zkb_fr_t* d_a, size_t d0, size_t d1,
                       const zkb_fr_t* h_u0, unsigned k0, const zkb_fr_t* h_u1, unsigned k1,
                       zkb_fr_t* h_out, void* stream);

/* ---- layout (fr-tensor.cu:800-828, 885-900) -------------------------------------- */
/* one level of FrTensor::pad (fr-tensor.cu:800-828): [rows, last] -> [rows, last_padded]
 * filled with pad_val */
int zkb_fr_pad_last(const zkb_fr_t* d_a, size_t rows, size_t last, size_t last_padded,
                    const zkb_fr_t* h_pad_val, zkb_fr_t* d_out, void* stream);
/* FrTensor::split (fr-tensor.cu:562-585): windows 0,2,4,.. go to d_out0 and 1,3,5,.. to
 * d_out1 (out_n elements each, zero past the end of the input) */
int zkb_fr_split_window(const zkb_fr_t* d_a, size_t n, size_t window, zkb_fr_t* d_out0, zkb_fr_t* d_out1,
                        size_t out_n, void* stream);
/* FrTensor::transpose (fr-tensor.cu:885-900): [M, N] -> [N, M] */
int zkb_fr_transpose(const zkb_fr_t* d_a, size_t M, size_t N, zkb_fr_t* d_out, void* stream);
/* FrTensor::matmul / zkFC::operator() (fr-tensor.cu:831-881, zkfc.cu:44-58):
 * C[M,P] = A[M,N] * B[N,P] over Fr */
int zkb_fr_matmul(const zkb_fr_t* d_a, const zkb_fr_t* d_b, zkb_fr_t* d_c,
                  size_t M, size_t N, size_t P, void* stream);
/* fcAddBiasKernel (zkfc.cu:36-41) */
int zkb_fr_add_bias(zkb_fr_t* d_z, const zkb_fr_t* d_bias, size_t rows, size_t cols, void* stream);

/* ---- sumchecks -------------------------------------------------------------------- */
/* zkip (zkfc.cu:94-151): inner-product sumcheck of two length-n vectors, pairing
 * (i, i + N/2) and consuming h_u from the back.  h_polys receives 3 coefficients
 * per round (k rounds, round 0 first); *h_final is the returned claim.  Returns
 * ZKB_ERR_VERIFY when a round fails claim == p(0) + p(1) ("claim != p(0) + p(1)").
 * The inputs are not modified. */
int zkb_zkip(const zkb_fr_t* h_claim, const zkb_fr_t* d_a, const zkb_fr_t* d_b, size_t n,
             const zkb_fr_t* h_u, unsigned k, zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream);
/* zkip_stacked (zkfc.cu:153-228): A and B are [num, D] tensors (one vector pair per layer or head).  kN =
 * ceilLog2(num) rounds over the stack - each weighted by eq over the remaining lower half of the stack, paired with
 * h_uN[kN - 1 - r] and folded with h_vN[kN - 1 - r] - then zkip over D with h_uD.  h_polys receives 3 coefficients
 * per round (kN + kD rounds); ZKB_ERR_VERIFY with "claim != q(0) + q(1)" (a stack round) or "claim != p(0) + p(1)". */
int zkb_zkip_stacked(const zkb_fr_t* h_claim, const zkb_fr_t* d_A, const zkb_fr_t* d_B, size_t num, size_t D,
                     const zkb_fr_t* h_uN, const zkb_fr_t* h_vN, unsigned kN, const zkb_fr_t* h_uD, unsigned kD,
                     zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream);
/* The first `rounds` rounds of zkip (zkfc.cu:94-151) without the verifier replay: no counterpart
 * in the reference; the building block of the multi-GPU split, where a rank's sums
 * are only part of each round polynomial.  Round r uses h_u[k - 1 - r].
 * h_sums receives 3 coefficient sums per round; h_tail_a / h_tail_b receive the two
 * vectors as folded by the last of these rounds, 2^(ceilLog2(n) - rounds) entries each
 * (the inputs themselves, n entries, when rounds is 0). */
int zkb_zkip_partial(const zkb_fr_t* d_a, const zkb_fr_t* d_b, size_t n, const zkb_fr_t* h_u, unsigned k,
                     unsigned rounds, zkb_fr_t* h_sums, zkb_fr_t* h_tail_a, zkb_fr_t* h_tail_b, void* stream);
/* Body of zkFC::prove (zkfc.cu:61-87) with the challenge vectors passed in
 * (the reference draws them from random_vec).  X is [B, I], W is [I, O], Y is
 * [B, O].  Outputs: h_polys (3 * ceilLog2(I) coefficients), h_claims[4] =
 * {claim (Y at (u_batch,u_output)), final_claim, claim_X, claim_W}.
 * ZKB_ERR_VERIFY when claim_X*claim_W != final_claim ("Claim does not match"). */
int zkb_zkfc_prove(const zkb_fr_t* d_X, const zkb_fr_t* d_W, const zkb_fr_t* d_Y,
                   size_t B, size_t I, size_t O,
                   const zkb_fr_t* h_u_batch, const zkb_fr_t* h_u_input, const zkb_fr_t* h_u_output,
                   zkb_fr_t* h_polys, zkb_fr_t* h_claims, void* stream);
/* tLookup::prep (tlookup.cu:23-48): multiplicities of `indices` in a table of N */
int zkb_tlookup_prep(const uint32_t* d_indices, size_t D, size_t N, zkb_fr_t* d_m, void* stream);
/* tLookupRange::prep(FrTensor) (tlookup.cu:414-433): index = low limb of (v - low) */
int zkb_tlookup_range_indices(const zkb_fr_t* d_vals, int32_t low, uint32_t* d_indices, size_t D, void* stream);
/* tLookupRange ctor (tlookup.cu:372-391): table of `table_size` (a power of two)
 * entries low, low+1, ..., repeating the last of the first `len` */
int zkb_tlookup_range_table(int32_t low, size_t len, size_t table_size, zkb_fr_t* d_table, void* stream);
/* lookuprangemapping_kernel (tlookup.cu:446-453): out[i] = vals[indices[i]] */
int zkb_fr_gather(const uint32_t* d_indices, const zkb_fr_t* d_vals, zkb_fr_t* d_out, size_t D, void* stream);
/* tLookup::prove (tlookup.cu:324-370 with phases :184-320).  S has D elements,
 * table and m have N; D and N powers of two, N | D; u and v have log2(D)
 * values.  h_polys receives 4 coefficients per round (log2 D rounds; the
 * reference computes these and drops them); *h_final is the returned claim.
 * ZKB_ERR_VERIFY: "tLookup_phase1: claim != p(0) + p(1)" / "tLookup_phase2: ...". */
int zkb_tlookup_prove(const zkb_fr_t* d_S, const zkb_fr_t* d_table, const zkb_fr_t* d_m,
                      size_t D, size_t N, const zkb_fr_t* h_alpha, const zkb_fr_t* h_beta,
                      const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                      zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream);
/* The same proof when the caller knows where each looked-up value sits in the table: d_indices[i]
 * (may be NULL) claims table[d_indices[i]] == S[i], as tLookupRange::prep computes it
 * (tlookup.cu:414-433).  A = 1/(S + beta) (tlookup.cu:50-62, 330) is then read from the N inverses
 * of the table instead of D inversions, inside the first round; a value that is not at its
 * claimed index is inverted on its own, so the transcript never depends on the indices. */
int zkb_tlookup_prove_indexed(const zkb_fr_t* d_S, const uint32_t* d_indices, const zkb_fr_t* d_table, const zkb_fr_t* d_m,
                              size_t D, size_t N, const zkb_fr_t* h_alpha, const zkb_fr_t* h_beta,
                              const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                              zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream);
/* The first `rounds` rounds of the same proof without the assembly of the round
 * polynomials and the verifier replay (tlookup.cu:281-322; no counterpart in the reference:
 * the building block of the multi-GPU split).  h_sums receives 1 + 11 * rounds values:
 * sum B*m, then per round [0..2] the eq-weighted (A,S) coefficients, phase 1: [3] sum A0,
 * [4] sum (A1 - A0); phase 2: [3..5] the eq-weighted (B,T) coefficients, [6] sum A0,
 * [7] sum (A1 - A0), [8..10] the coefficients of (m0 + m1 t)(B0 + B1 t).  h_tails receives
 * A, S (D >> rounds entries each) and B, T, m (N >> max(rounds - log2(D/N), 0) each) as the
 * last of these rounds left them. */
int zkb_tlookup_partial(const zkb_fr_t* d_S, const zkb_fr_t* d_table, const zkb_fr_t* d_m, size_t D, size_t N,
                        const zkb_fr_t* h_beta, const zkb_fr_t* h_u, const zkb_fr_t* h_v, unsigned rounds,
                        zkb_fr_t* h_sums, zkb_fr_t* h_tails, void* stream);
/* The exchange step of the multi-GPU split (no counterpart in the reference; zkfc.cu:140-151 and
 * tlookup.cu:281-322 are the checks replayed here).  The vectors are dealt out round-robin, rank p
 * holding the indices p, p + world, ...; every rank has run all its local rounds and h_parts holds
 * the `world` gathered blocks in rank order.  Pure host arithmetic.
 * zkip: block = 3 * (k - log2 world) coefficient sums, then the rank's surviving pair (a, b);
 *   h_polys receives 3 * k coefficients.
 * tLookup: block = the 1 + 11 * (log2 D - log2 world) sums of zkb_tlookup_partial, then the rank's
 *   surviving A, S, B, T, m; h_u, h_v are the challenges of the whole proof; h_polys receives
 *   4 * log2 D coefficients.  Both return ZKB_ERR_VERIFY with the reference's message when a round
 *   does not verify. */
int zkb_zkip_combine(const zkb_fr_t* h_parts, unsigned world, unsigned k, const zkb_fr_t* h_u, const zkb_fr_t* h_claim,
                     zkb_fr_t* h_polys, zkb_fr_t* h_final);
int zkb_tlookup_combine(const zkb_fr_t* h_parts, unsigned world, size_t D, size_t N, const zkb_fr_t* h_alpha,
                        const zkb_fr_t* h_beta, const zkb_fr_t* h_u, const zkb_fr_t* h_v, zkb_fr_t* h_polys,
                        zkb_fr_t* h_final);
/* multi_hadamard_sumchecks (proof.cu:190-241): K tensors of N (a power of two)
 * elements; h_polys receives (K+1) coefficients per round, log2 N rounds. */
int zkb_multi_hadamard(const zkb_fr_t* h_claim, const zkb_fr_t* const* h_d_Xs, unsigned K, size_t N,
                       const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                       zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream);
/* All log2 N rounds of the same proof without the verifier replay (proof.cu:190-241; no counterpart in the
 * reference: the building block of the multi-GPU split).  h_sums receives the (K+1) coefficient sums of every
 * round, h_tails the K entries that are left (the inputs themselves when N is 1). */
int zkb_multi_hadamard_partial(const zkb_fr_t* const* h_d_Xs, unsigned K, size_t N, const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                               zkb_fr_t* h_sums, zkb_fr_t* h_tails, void* stream);
/* The exchange step of the split multi_hadamard_sumchecks (no counterpart in the reference; proof.cu:190-241 are the
 * checks replayed).  The K tensors of 2^kN entries are dealt out round-robin; rank p has run zkb_multi_hadamard_partial
 * on its share with the challenges h_u + log2 world, h_v + log2 world.  h_parts holds the `world` blocks in rank
 * order: (kN - log2 world) * (K+1) sums, then the rank's K surviving entries.  The sums are weighted by eq(u; p) over
 * the rank's index bits and added, the last log2 world rounds run here on the surviving entries; h_polys receives
 * (K+1) * kN coefficients.  Pure host arithmetic; ZKB_ERR_VERIFY with the reference's message when a round fails. */
int zkb_multi_hadamard_combine(const zkb_fr_t* h_parts, unsigned world, unsigned K, unsigned kN, const zkb_fr_t* h_u,
                               const zkb_fr_t* h_v, const zkb_fr_t* h_claim, zkb_fr_t* h_polys, zkb_fr_t* h_final);
/* hadamard_product_sumcheck / inner_product_sumcheck / binary_sumcheck
 * (proof.cu:12-160), including the factor 2^-256 the reference leaves on the
 * product terms.  h_proof receives 3*k + 2 (3*k + 1 for binary) elements. */
int zkb_hadamard_product_sumcheck(const zkb_fr_t* d_a, const zkb_fr_t* d_b, size_t n,
                                  const zkb_fr_t* h_u, const zkb_fr_t* h_v, unsigned k,
                                  zkb_fr_t* h_proof, void* stream);
int zkb_inner_product_sumcheck(const zkb_fr_t* d_a, const zkb_fr_t* d_b, size_t n,
                               const zkb_fr_t* h_u, unsigned k, zkb_fr_t* h_proof, void* stream);
int zkb_binary_sumcheck(const zkb_fr_t* d_a, size_t n, const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                        unsigned k, zkb_fr_t* h_proof, void* stream);

/* ---- Rescaling / softmax element kernels ------------------------------------------ */
/* rescaling_kernel (rescaling.cu:8-21): out = round-to-nearest x / sf, rem = x - out*sf
 * in [-sf/2, sf/2) */
int zkb_rescale(const zkb_fr_t* d_in, uint64_t scaling_factor, zkb_fr_t* d_out, zkb_fr_t* d_rem,
                size_t n, void* stream);
/* zkrelu_decomp_kernel (zkrelu.cu:9-30): with q = round-to-nearest x / sf as above,
 * sign = (q >= 0), abs = |q|, rem = x - q*sf, res = max(q, 0) */
int zkb_relu_decomp(const zkb_fr_t* d_in, uint64_t scaling_factor, zkb_fr_t* d_sign, zkb_fr_t* d_abs,
                    zkb_fr_t* d_rem, zkb_fr_t* d_res, size_t n, void* stream);
/* zksoftmax_calculate_table (zksoftmax.cu:4-16) */
int zkb_softmax_table(double theta_k, double scaling_factor_in, double d, double Bk, uint32_t bk,
                      zkb_fr_t* d_table, void* stream);
/* zksoftmax_shift (zksoftmax.cu:20-32): per row shift = round(sf*sqrt(d)*ln(sum exp(x/(sf*sqrt(d)))))
 * with the row sum taken left to right in double precision; out = A - shift */
int zkb_softmax_shift(const zkb_fr_t* d_A, zkb_fr_t* d_shift, zkb_fr_t* d_out, size_t rows, size_t cols,
                      double scaling_factor_in, double d, void* stream);
/* zksoftmax_decompose_kernel (zksoftmax.cu:95-109): mixed-radix digits of -X,
 * digit i of element g stored at d_out[i*N + g] */
int zkb_softmax_decompose(const zkb_fr_t* d_X, const uint32_t* h_bs, unsigned K, zkb_fr_t* d_out,
                          size_t N, void* stream);

/* ---- G1 tensors: fills, negation, elementwise and broadcast add/sub, affine lift
 *      (g1-tensor.cu:61-375) -------------------------------------------------------------- */
int zkb_g1_fill(zkb_g1_t* d_out, const zkb_g1_t* h_val, size_t n, void* stream);
int zkb_g1_neg(const zkb_g1_t* d_a, zkb_g1_t* d_out, size_t n, void* stream);
int zkb_g1_add(const zkb_g1_t* d_a, const zkb_g1_t* d_b, zkb_g1_t* d_out, size_t n, void* stream);
int zkb_g1_sub(const zkb_g1_t* d_a, const zkb_g1_t* d_b, zkb_g1_t* d_out, size_t n, void* stream);
int zkb_g1_add_scalar(const zkb_g1_t* d_a, const zkb_g1_t* h_x, zkb_g1_t* d_out, size_t n, void* stream);
int zkb_g1_from_affine(const zkb_g1_affine_t* d_a, zkb_g1_t* d_out, size_t n, void* stream);
/* Jacobian -> affine (X/Z^2, Y/Z^3), identity -> (0,0).  It has no counterpart in the
 * reference: this is the normal form on which G1 results are compared. */
int zkb_g1_to_affine(const zkb_g1_t* d_a, zkb_g1_affine_t* d_out, size_t n, void* stream);
/* G1TensorJacobian::operator*(FrTensor) (g1-tensor.cu:445-480): out[i] = scalars[i] * g[i mod n_g] */
int zkb_g1_mul(const zkb_g1_t* d_g, size_t n_g, const zkb_fr_t* d_scalars, size_t n, zkb_g1_t* d_out, void* stream);
/* G1TensorJacobian::sum (g1-tensor.cu:391-443) */
int zkb_g1_sum(const zkb_g1_t* d_a, size_t n, zkb_g1_t* h_out, void* stream);
/* G1TensorJacobian::rowwise_sum (g1-tensor.cu:535-625) */
int zkb_g1_rowwise_sum(const zkb_g1_t* d_a, size_t rows, size_t cols, zkb_g1_t* d_out, void* stream);
/* G1TensorJacobian::operator()(u) (g1-tensor.cu:486-514).  The reference passes u
 * through an un-Montgomery step first (g1-tensor.cu:491); reproduced. */
int zkb_g1_mle_eval(const zkb_g1_t* d_a, size_t n, const zkb_fr_t* h_u, unsigned k, zkb_g1_t* h_out, void* stream);

/* ---- commitment (commitment.cu) ----------------------------------------------------- */
/* Commitment::commit_int (commitment.cu:31-58): m = n_scalars / n_gen row
 * commitments; scalars are Fr encodings of int32 values. */
int zkb_commit_int(const zkb_g1_t* d_gens, size_t n_gen, const zkb_fr_t* d_scalars, size_t n_scalars,
                   zkb_g1_t* d_out, void* stream);
/* Same with the scalars given directly as int32 (the weight .bin format,
 * fileio_utils.py:4-12; read by FrTensor::from_int_bin, fr-tensor.cu:226-236): skips the
 * 8x larger Fr encoding. */
int zkb_commit_i32(const zkb_g1_t* d_gens, size_t n_gen, const int32_t* d_scalars, size_t n_scalars,
                   zkb_g1_t* d_out, void* stream);
/* Same call with the algorithm prescribed instead of chosen by the library's cost estimate
 * (commitment.cu:31-58 has one algorithm; both of these return the same group elements):
 * ZKB_MSM_BUCKETS - bucket method, signed 7-bit windows, best for few rows or many generators;
 * ZKB_MSM_TABLES  - per-call tables of all digit combinations of four generators, signed 3-bit
 *                   windows, best for many rows over one generator set (96 bytes * 1024 per
 *                   generator of scratch memory). */
#define ZKB_MSM_AUTO 0
#define ZKB_MSM_BUCKETS 1
#define ZKB_MSM_TABLES 2
int zkb_commit_i32_method(const zkb_g1_t* d_gens, size_t n_gen, const int32_t* d_scalars, size_t n_scalars,
                          zkb_g1_t* d_out, int method, void* stream);
/* Host-buffer form of the same call - what commit-param.cu:12-28 does through files:
 * copies generators and int32 scalars in, commits, copies the m Jacobian results out. */
int zkb_commit_i32_host(const zkb_g1_t* h_gens, size_t n_gen, const int32_t* h_scalars, size_t n_scalars,
                        zkb_g1_t* h_out, void* stream);
/* Commitment::commit (commitment.cu:22-29): full-width scalars */
int zkb_commit(const zkb_g1_t* d_gens, size_t n_gen, const zkb_fr_t* d_scalars, size_t n_scalars,
               zkb_g1_t* d_out, void* stream);
/* Commitment::me_open (commitment.cu:79-129): t and generators have n elements,
 * k challenges.  h_proof receives 3*k + 1 Jacobian points (the reference builds
 * this vector and drops it); *h_out is the opening. */
int zkb_me_open(const zkb_fr_t* d_t, const zkb_g1_t* d_gens, size_t n, const zkb_fr_t* h_u, unsigned k,
                zkb_g1_t* h_proof, zkb_fr_t* h_out, void* stream);
/* The same opening in two halves (no counterpart in the reference, whose me_open returns when it is done;
 * commitment.cu:111-125 is what both halves compute).  zkb_me_open_begin orders the opening after the work already
 * queued on `stream`, queues it on streams of its own and returns a handle; zkb_me_open_end waits for it, writes
 * the 3 k + 1 proof elements and the opening, and releases the handle (call it exactly once per handle, also after
 * an error elsewhere).  d_t and d_gens must stay as they are until then; h_u is read during begin only.  Up to four
 * openings per device run side by side with whatever the caller queues meanwhile; a further begin runs its opening at
 * once and end only hands over the results. */
int zkb_me_open_begin(const zkb_fr_t* d_t, const zkb_g1_t* d_gens, size_t n, const zkb_fr_t* h_u, unsigned k, void* stream,
                      void** handle);
int zkb_me_open_end(void* handle, zkb_g1_t* h_proof, zkb_fr_t* h_out);

/* ---- multi-GPU: one process per GPU (no counterpart in the reference, which is single-GPU) ----
 * The process's communicator is an NCCL communicator on the device that is current when
 * zkb_comm_init runs; rank 0 makes the 128-byte id (zkb_comm_unique_id) and hands it to the other
 * ranks by any means (a file, MPI, torch.distributed).  Every exchange is a plain all-gather
 * on this GPU's own buffers.  The sharded provers below do all their local work first and
 * exchange once; every rank returns the same result as the single-GPU call on the whole data. */
int zkb_comm_unique_id(unsigned char* id128);
int zkb_comm_init(int rank, int world, const unsigned char* id128);
int zkb_comm_info(int* rank, int* world);               /* world == 0: not initialised */
int zkb_comm_destroy(void);
/* d_recv[p * bytes_per_rank ...] = rank p's d_send; queued on the stream, no host synchronisation
 * (no counterpart in the reference) */
int zkb_comm_allgather(const void* d_send, void* d_recv, size_t bytes_per_rank, void* stream);
/* Commitment::commit_int (commitment.cu:31-58) with the rows dealt out in contiguous blocks: rank p
 * holds rows [p*m/P ..) (the first m % P ranks one row more) as int32, the generators are on
 * every rank, d_out_all receives all rows_total commitments in row order on every rank. */
int zkb_commit_i32_sharded(const zkb_g1_t* d_gens, size_t n_gen, const int32_t* d_scalars_local, size_t rows_local,
                           size_t rows_total, zkb_g1_t* d_out_all, void* stream);
/* The same commitments with the COLUMNS dealt out instead: rank p holds a contiguous block of the
 * generators and, for all `rows` rows, the scalars of those columns (rows x n_gen_local, int32).  Every rank
 * commits its block (the per-call tables of the generators are then built for n / P generators only),
 * the P partial commitments of each row are all-gathered and added in rank order; d_out receives the
 * `rows` commitments on every rank - the same group elements as commitment.cu:31-58 on the whole matrix. */
int zkb_commit_i32_colsharded(const zkb_g1_t* d_gens_local, size_t n_gen_local, const int32_t* d_scalars_local, size_t rows,
                              zkb_g1_t* d_out, void* stream);
/* zkFC::prove's body (zkfc.cu:61-87) with W dealt out by rows round-robin and X by the matching
 * columns: rank p holds X[:, p::P] (B x I_local) and W[p::P, :] (I_local x O), Y is on every rank.
 * h_u_input has log2(I_local * P) entries.  Outputs as zkb_zkfc_prove. */
int zkb_zkfc_prove_sharded(const zkb_fr_t* d_X_local, const zkb_fr_t* d_W_local, const zkb_fr_t* d_Y,
                           size_t B, size_t I_local, size_t O,
                           const zkb_fr_t* h_u_batch, const zkb_fr_t* h_u_input, const zkb_fr_t* h_u_output,
                           zkb_fr_t* h_polys, zkb_fr_t* h_claims, void* stream);
/* tLookup::prove (tlookup.cu:324-370) with S, the table and the multiplicities dealt out round-robin:
 * rank p holds S[p::P], T[p::P], m[p::P]; D, N and the challenges are those of the whole proof. */
int zkb_tlookup_prove_sharded(const zkb_fr_t* d_S_local, const zkb_fr_t* d_table_local, const zkb_fr_t* d_m_local,
                              size_t D, size_t N, const zkb_fr_t* h_alpha, const zkb_fr_t* h_beta,
                              const zkb_fr_t* h_u, const zkb_fr_t* h_v,
                              zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream);
/* multi_hadamard_sumchecks (proof.cu:190-241) with the K tensors dealt out round-robin: rank p holds X_k[p::P]
 * (N / P entries each); N, the claim and the challenges are those of the whole proof.  Outputs as
 * zkb_multi_hadamard, on every rank. */
int zkb_multi_hadamard_sharded(const zkb_fr_t* h_claim, const zkb_fr_t* const* h_d_Xs_local, unsigned K, size_t N,
                               const zkb_fr_t* h_u, const zkb_fr_t* h_v, zkb_fr_t* h_polys, zkb_fr_t* h_final, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ZKLLM_B200_H */
