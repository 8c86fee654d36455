/* zkb200 - C ABI of the B200 proving hot path (BN254 sumcheck provers, multilinear folds,
 * KZH2/KZH3 commit/open multi-scalar multiplications).
 *
 * The reference (crate zk_torch_2) has no FFI for this path; its seams are Rust traits.  Each
 * entry point below names the reference function it stands in for (paths relative to the
 * reference crate root).  A Rust shim implements the traits on top of these calls.
 *
 * Conventions
 *  - Fr / Fq elements cross the boundary as 4 x uint64_t little-endian limbs in Montgomery form
 *    (a * 2^256 mod p): byte-identical to arkworks' in-memory Fp256, so a Vec<Fr> can be passed
 *    by pointer.
 *  - G1 affine points are {x[4], y[4]} (64 bytes, Montgomery mod q); the point at infinity is
 *    encoded as x = y = 0 (not on the curve, so unambiguous).
 *  - G1 projective results are Jacobian {X[4], Y[4], Z[4]} (96 bytes), Z = 0 for infinity;
 *    compare after normalising, as with arkworks' Projective.
 *  - Every function returns ZK_OK (0) or a negative zk_status; zk_last_error() gives the
 *    message of the calling thread's last failure.  A Rust shim turns a non-zero status into
 *    the panic / Err(String) the trait in question documents.
 *  - `mem` arguments say where a caller buffer lives: ZK_MEM_HOST or ZK_MEM_DEVICE (a CUDA
 *    device pointer on the context's GPU).  Inputs are never modified.
 *  - A zk_ctx may be shared by host threads, as the reference opens its commitments from many rayon workers at
 *    once (src/dag/mod.rs:893-936): up to ZK_OPT_LANES calls run concurrently, each on a stream and scratch of
 *    its own; SRS handles and caller buffers are shared and only read.  Sharded calls (a zk_comm) and the calls
 *    that read the context's statistics take the first lane and are serialised among themselves.
 */
#ifndef ZKB200_H
#define ZKB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct zk_ctx zk_ctx;
typedef struct zk_transcript zk_transcript;
typedef struct zk_comm zk_comm;

typedef enum zk_status {
  ZK_OK = 0,
  ZK_ERR_ARG = -1,         /* shape / argument errors: the reference's assert! panics */
  ZK_ERR_OOM = -2,         /* device allocation failed */
  ZK_ERR_CUDA = -3,        /* a CUDA call or kernel failed */
  ZK_ERR_TIMEOUT = -4,     /* a bounded device-side wait ran out */
  ZK_ERR_FS_CALLBACK = -5, /* the caller's Fiat-Shamir callback returned non-zero */
  ZK_ERR_COMM = -6         /* multi-GPU exchange failed */
} zk_status;

typedef enum zk_mem { ZK_MEM_HOST = 0, ZK_MEM_DEVICE = 1 } zk_mem;

#define ZK_MAX_POLYS 4

/* ---- context ------------------------------------------------------------------------- */
/* One context per GPU (and per process rank).  No counterpart in the reference: it holds
 * the stream and scratch that rayon's global pool and Vec allocations stand for there. */
int zk_init(int device, zk_ctx** out);
void zk_free(zk_ctx* ctx);
const char* zk_last_error(void);
/* Number of kernels this library has launched on the context since it was created. */
uint64_t zk_launch_count(const zk_ctx* ctx);
/* Options.  ZK_OPT_DEVICE_TAIL (default 1): the dense provers hand the rounds at or below 1024
 * table entries to one resident block that also runs the built-in transcript on the device
 * (identical outputs; only taken without a Fiat-Shamir callback and outside sharded rounds).
 * 0 keeps every round on the per-round kernels with the transcript on the host.
 * ZK_OPT_REPLICATE_LOG (default 18): a sharded dense round loop gathers the tables onto every rank once all
 * ranks together hold at most 2^value entries per table and finishes there without further exchanges
 * (identical outputs); 0 keeps every local round sharded.
 * ZK_OPT_PEER_EXCHANGE (default 1): sharded proves exchange the per-round partial sums through peer memory
 * (one kernel per round that stores into every rank's box over NVLink and waits, bounded, for the others'
 * shares) when zk_comm_init could map the ranks' boxes; 0 uses the NCCL all-gather (identical outputs).  Set it
 * to the same value on every rank.
 * ZK_OPT_EXCHANGE_WAIT_MS (default 16000): roughly how long a kernel of a sharded prove waits for another
 * rank's words before it gives up and the call returns ZK_ERR_TIMEOUT (the ranks are separate processes and
 * may reach a call seconds apart; a service with tight deadlines, or a test, sets it lower).
 * ZK_OPT_LANES (default 4): how many calls on this context may run at the same time.  Each concurrent call gets a
 * lane of its own (a stream and grow-only scratch, created when a second, third ... thread first arrives and kept
 * until zk_free); further callers wait for a free lane.  A single-threaded host only ever uses the first lane.
 * ZK_OPT_AHEAD_LOG (default 15): an unsharded dense prove with the built-in transcript and at most three tables runs
 * in one launch; once its tables are down to 2^value entries (four times that for a single table), each message is
 * tabulated as a polynomial in the challenge before it while that challenge is still being hashed (identical
 * outputs).  0 keeps every round in step and hands the last rounds to the single-block kernel. */
typedef enum zk_option {
  ZK_OPT_DEVICE_TAIL = 1, ZK_OPT_REPLICATE_LOG = 2, ZK_OPT_PEER_EXCHANGE = 3, ZK_OPT_EXCHANGE_WAIT_MS = 4, ZK_OPT_LANES = 5,
  ZK_OPT_AHEAD_LOG = 6
} zk_option;
int zk_set_option(zk_ctx* ctx, int option, int value);
/* Diagnostics: the host clock, in microseconds from the first entry, at which each round that the host steps
 * (a caller's transcript, the entry-form rounds of the sparse provers, sharded rounds) had its challenge, for
 * the proves since the last call (at most 4096 entries are kept).  Writes up to cap entries, sets *n to the
 * number recorded and clears the record.  Rounds that run inside the resident kernels leave no entry.  The
 * sparse x dense prover also marks its entry, the return of its dense rounds and its exit.  No counterpart in the
 * reference. */
int zk_round_times(zk_ctx* ctx, double* out_us, uint32_t cap, uint32_t* n);
/* The CUDA stream (cudaStream_t) every kernel of this context is launched on, so a host can
 * bracket calls with its own events. */
void* zk_stream(zk_ctx* ctx);
/* Per-kernel-kind device timing (CUDA events on the context's stream around each launch).
 * Enabling clears the totals.  zk_profile_get synchronises the stream and returns, for one
 * kind, the launches, their summed duration and their summed algorithmic bytes. */
typedef enum zk_prof_kind {
  ZK_PROF_ROUND = 0,       /* dense round kernel (fold + message) */
  ZK_PROF_FOLD = 1,        /* plain LSB fold */
  ZK_PROF_SPARSE_MSG = 2,  /* round message over sparse entries */
  ZK_PROF_SPARSE_FOLD = 3, /* entry fold + compaction (3 launches per round) */
  ZK_PROF_FROM_RIGHT = 4,  /* fix_variables_from_right / eq tables */
  ZK_PROF_MSM = 5,         /* multi-scalar multiplication pipeline */
  ZK_PROF_OTHER = 6
} zk_prof_kind;
int zk_profile_enable(zk_ctx* ctx, int on);
int zk_profile_get(zk_ctx* ctx, int kind, uint64_t* launches, double* ms, double* bytes);
/* Device memory owned by the caller (thin cudaMalloc / cudaFree / cudaMemcpy wrappers for
 * hosts that do not link the CUDA runtime themselves). */
int zk_device_alloc(zk_ctx* ctx, size_t bytes, void** out);
int zk_device_free(zk_ctx* ctx, void* ptr);
int zk_device_copy(zk_ctx* ctx, void* dst, zk_mem dst_mem, const void* src, zk_mem src_mem, size_t bytes);
int zk_device_sync(zk_ctx* ctx);

/* ---- Fiat-Shamir transcript: src/util/transcript.rs:13-46 (merlin 3.0.0) -------------- */
zk_transcript* zk_transcript_new(const uint8_t* label, size_t label_len);     /* Transcript::new */
zk_transcript* zk_transcript_clone(const zk_transcript* t);                   /* #[derive(Clone)] */
void zk_transcript_free(zk_transcript* t);
void zk_transcript_append_message(zk_transcript* t, const uint8_t* label, size_t label_len, const uint8_t* msg,
                                  size_t msg_len);                            /* :19-21 */
void zk_transcript_append_u64(zk_transcript* t, const uint8_t* label, size_t label_len, uint64_t value); /* :23-25 */
void zk_transcript_append_scalar(zk_transcript* t, const uint8_t* label, size_t label_len,
                                 const uint64_t scalar[4]);                   /* :27-30, Montgomery in */
void zk_transcript_challenge_bytes(zk_transcript* t, const uint8_t* label, size_t label_len, uint8_t* out,
                                   size_t n);
void zk_transcript_challenge_scalar(zk_transcript* t, const uint8_t* label, size_t label_len,
                                    uint64_t out[4]);                         /* :38-42, Montgomery out */

/* Per-round Fiat-Shamir callback, for callers that keep their own transcript (the Rust shim
 * passes the real merlin crate through this).  msgs: n_msgs round-message scalars; the
 * callback absorbs them and writes the round challenge.  Return 0 on success. */
typedef int (*zk_fs_round_fn)(void* user, const uint64_t* msgs, uint32_t n_msgs, uint64_t challenge_out[4]);

/* ---- sumcheck provers ----------------------------------------------------------------- */
/* LinearSumcheckProver::prove, src/crypto/sumcheck/linear_prover.rs:43-76 (rounds :82-178,
 * final :181-190).  The header (num_var, num_poly) is absorbed by the caller as ::new does
 * (:29-41).  tables: num_poly pointers to 2^num_var elements each.  With fs == NULL the
 * built-in transcript `tr` absorbs each message scalar under "round_message" and draws
 * "challenge".  Outputs (host): round_msgs[num_var][num_poly+1], challenges[num_var],
 * final_table0[num_poly] (= a_arrays[i][0] after the last round), final_eval. */
int zk_sumcheck_linear_prove(zk_ctx* ctx, uint32_t num_var, uint32_t num_poly, const uint64_t* const* tables,
                             zk_mem tables_mem, zk_fs_round_fn fs, void* fs_user, zk_transcript* tr,
                             uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_table0,
                             uint64_t* final_eval);

/* Product sumcheck sum_x a(x) b(x) with `a` given by nnz non-zero entries (idx strictly
 * increasing, < 2^num_var; vals their values) and `b` a dense table of 2^num_var elements.
 * The reference has no prover of this shape in src/ (tests/test_sd_sumcheck.rs:46-58 imports
 * a missing module); the result is defined as LinearSumcheckProver::prove
 * (linear_prover.rs:43-76) on [a.to_dense(), b]: same messages (3 per round), challenges,
 * final_table0 = {a(r), b(r)} and final_eval.  All three inputs live in `mem`.  num_var <= 32. */
int zk_sumcheck_sparse_dense_prove(zk_ctx* ctx, uint32_t num_var, uint64_t nnz, const uint64_t* idx,
                                   const uint64_t* vals, const uint64_t* dense, zk_mem mem, zk_fs_round_fn fs,
                                   void* fs_user, zk_transcript* tr, uint64_t* round_msgs, uint64_t* challenges,
                                   uint64_t* final_table0, uint64_t* final_eval);

/* SparseBoolSumcheckProver::prove, src/crypto/sumcheck/linear_prover.rs:486-656 (header
 * num_var, num_poly = 3 absorbed by the caller as ::new does, :468-478): proves
 * sum_x eq(eq_point, x) sum_j weights[j] s_j(x) (s_j(x) - 1) with s_j the 0/1 selection table whose
 * ones are term j's positions.  positions: the terms' position lists concatenated (any order
 * inside a term, distinct; n_positions[j] entries for term j).  Host inputs.  Outputs:
 * round_msgs[num_var][4], challenges[num_var], final_eval. */
int zk_sumcheck_sparse_bool_prove(zk_ctx* ctx, uint32_t num_var, uint32_t n_terms, const uint64_t* weights,
                                  const uint64_t* positions, const uint64_t* n_positions, const uint64_t* eq_point,
                                  zk_fs_round_fn fs, void* fs_user, zk_transcript* tr, uint64_t* round_msgs,
                                  uint64_t* challenges, uint64_t* final_eval);
/* GeneralLinearSumcheckProver::prove, linear_prover.rs:229-438: sum_x eq(x) sum_j scalars[j]
 * prod_i p_ji(x).  num_poly counts eq as one factor (:233), so every term has num_poly - 1 tables;
 * tables[j * (num_poly - 1) + i] = p_ji, eq = the eq table, all 2^num_var elements in `mem`.
 * Outputs: round_msgs[num_var][num_poly + 1], challenges, final_tables[n_terms * (num_poly - 1)]
 * (every table's fully bound value; may be NULL), final_eval. */
int zk_sumcheck_general_prove(zk_ctx* ctx, uint32_t num_var, uint32_t num_poly, uint32_t n_terms, const uint64_t* scalars,
                              const uint64_t* const* tables, const uint64_t* eq, zk_mem mem, zk_fs_round_fn fs,
                              void* fs_user, zk_transcript* tr, uint64_t* round_msgs, uint64_t* challenges,
                              uint64_t* final_tables, uint64_t* final_eval);

/* SumcheckVerifier::verify, src/crypto/sumcheck/verifier.rs:27-69 (the header num_var, num_poly is absorbed
 * by the caller as ::new does, :14-17): checks every round's s(0) + s(1) against the running sum, absorbs the
 * evaluations, draws the challenge and interpolates (evaluate_univariate_polynomial, src/util/poly.rs:446-563).
 * Host arithmetic only, no device is touched.  round_msgs: n_rounds x msgs_per_round elements.  *accepted = 1
 * with the last running sum in final_sum_out (the caller compares it with the product of the tables' values at
 * the challenges) and the challenges in challenges_out (either may be NULL); *accepted = 0 where the reference
 * returns (None, vec![]): a wrong round count, a wrong number of evaluations, or a round that does not continue
 * the running sum (its index in *failed_round, optional). */
int zk_sumcheck_verify(zk_transcript* tr, uint32_t num_var, uint32_t num_poly, const uint64_t* round_msgs,
                       uint32_t n_rounds, uint32_t msgs_per_round, const uint64_t* claimed_sum,
                       uint64_t* challenges_out, uint64_t* final_sum_out, int* accepted, uint32_t* failed_round);

/* ---- multi-GPU (one process per GPU; no counterpart in the reference, which is single-process) --- */
/* A communicator over `world` ranks (a power of two, at most 64), bound to NCCL at run time.
 * Rank 0 calls zk_comm_unique_id and the host distributes the 128 bytes to the other ranks. */
int zk_comm_unique_id(uint8_t out[128]);
/* Error contract of the sharded calls below (every entry point that takes a zk_comm): they are collective,
 * every rank makes the same calls in the same order.  When one of them returns non-zero on a rank, the
 * communicator is retired on that rank: the ranks may have parted mid-exchange (one returned early, the
 * others ran into a bounded wait and returned ZK_ERR_TIMEOUT), so every later sharded call on it returns
 * ZK_ERR_COMM at once, without launching anything, until the host calls zk_comm_free and zk_comm_init
 * again on all ranks.  A prove therefore either succeeds on every rank or fails on every rank, and a stale
 * share of an aborted round is never taken for a fresh one. */
int zk_comm_init(zk_ctx* ctx, int rank, int world, const uint8_t unique_id[128], zk_comm** out);
void zk_comm_free(zk_ctx* ctx, zk_comm* comm);
/* 1 when every rank of the communicator mapped every other rank's exchange box (CUDA IPC over NVLink peer
 * access) at zk_comm_init, so that ZK_OPT_PEER_EXCHANGE applies; 0 when the ranks stay on NCCL.  No counterpart
 * in the reference (single process). */
int zk_comm_peer_exchange(const zk_comm* comm);
/* Self-test of the bounded wait of the peer exchange on one GPU: runs the exchange kernel as rank 0 of two
 * with both boxes mapped to one scratch box, so that rank 1's share never arrives; the wait gives up after
 * `polls` polls (about a microsecond each, at most 2^22) and the call returns ZK_ERR_TIMEOUT, which is the
 * expected outcome; the context stays usable.  ZK_OK would mean the wait was satisfied by nothing.  No
 * counterpart in the reference. */
int zk_comm_wait_selftest(zk_ctx* ctx, uint32_t polls);
/* Sharded provers: the hypercube is cut on its top log2(world) variables, rank p holding entries
 * [p 2^num_var / world, (p+1) 2^num_var / world) of every table (for the sparse table: the
 * entries of that range, with indices relative to its start).  Each local round ends with an
 * all-gather of the ranks' partial round messages, summed on every rank; all ranks run
 * identical transcripts (pass equal-state transcripts or equivalent callbacks) and return
 * identical outputs, sized as for the unsharded call with the total num_var.  Once the local
 * variables are bound, the per-rank values are gathered and every rank finishes the last
 * log2(world) rounds on them. */
int zk_sumcheck_linear_prove_sharded(zk_ctx* ctx, zk_comm* comm, uint32_t num_var, uint32_t num_poly,
                                     const uint64_t* const* local_tables, zk_mem tables_mem, zk_fs_round_fn fs,
                                     void* fs_user, zk_transcript* tr, uint64_t* round_msgs, uint64_t* challenges,
                                     uint64_t* final_table0, uint64_t* final_eval);
int zk_sumcheck_sparse_dense_prove_sharded(zk_ctx* ctx, zk_comm* comm, uint32_t num_var, uint64_t local_nnz,
                                           const uint64_t* local_idx, const uint64_t* local_vals,
                                           const uint64_t* local_dense, zk_mem mem, zk_fs_round_fn fs, void* fs_user,
                                           zk_transcript* tr, uint64_t* round_msgs, uint64_t* challenges,
                                           uint64_t* final_table0, uint64_t* final_eval);
/* The boolean-check prover sharded by terms (the reference's prover is one loop over the terms,
 * linear_prover.rs:529-591: no counterpart of the split itself): every rank passes its own share of the terms
 * (weights, positions, n_positions as in zk_sumcheck_sparse_bool_prove; a rank may hold none), the same num_var and
 * eq_point, and an equal-state transcript.  The ranks' partial round messages and partial final values are summed
 * across the ranks; all ranks return the outputs of the unsharded call over all the terms. */
int zk_sumcheck_sparse_bool_prove_sharded(zk_ctx* ctx, zk_comm* comm, uint32_t num_var, uint32_t n_local_terms,
                                          const uint64_t* weights, const uint64_t* positions, const uint64_t* n_positions,
                                          const uint64_t* eq_point, zk_fs_round_fn fs, void* fs_user, zk_transcript* tr,
                                          uint64_t* round_msgs, uint64_t* challenges, uint64_t* final_eval);

/* MSM sharded by point range: every rank passes its own bases and scalars (n_local pairs), the
 * partial G1 sums are all-gathered and added; all ranks receive the same Jacobian point. */
int zk_msm_g1_sharded(zk_ctx* ctx, zk_comm* comm, const uint64_t* local_bases, zk_mem bases_mem,
                      const uint64_t* local_scalars, zk_mem scalars_mem, uint64_t n_local, uint64_t* out_jac);
/* fix_variables_from_right (src/util/poly.rs:705-758) over a table cut on its top log2(world)
 * variables: local_evals = the rank's 2^n / world entries, point binds the k highest variables
 * (k >= log2 world); every rank receives the whole 2^(n-k) result (host). */
int zk_fix_from_right_sharded(zk_ctx* ctx, zk_comm* comm, uint32_t n, const uint64_t* local_evals, zk_mem evals_mem,
                              uint32_t k, const uint64_t* point, uint64_t* out);

/* ---- multilinear helpers --------------------------------------------------------------- */
/* DenseMLPoly::fix_variables, src/util/poly.rs:842-887: binds the k lowest variables of a
 * 2^n table to point[0..k); out receives 2^(n-k) elements. */
int zk_fold_lsb(zk_ctx* ctx, uint32_t n, const uint64_t* evals, zk_mem evals_mem, uint32_t k, const uint64_t* point,
                uint64_t* out, zk_mem out_mem);

/* fix_variables_from_right, src/util/poly.rs:705-758: binds the k highest variables of a 2^n
 * table to point[0..k) (point[0] is variable n-k); out receives 2^(n-k) elements:
 * out[lo] = sum_hi eq(point)[hi] * evals[hi * 2^(n-k) + lo]. */
int zk_fix_from_right(zk_ctx* ctx, uint32_t n, const uint64_t* evals, zk_mem evals_mem, uint32_t k, const uint64_t* point,
                      uint64_t* out, zk_mem out_mem);
/* evaluate_multilinear_extension / DenseMLPoly::evaluate_at_point, src/util/poly.rs:622-652, 788-791:
 * out (4 x u64, host) = sum_i evals[i] * eq(i, point) for a table of 2^n elements and n coordinates. */
int zk_mle_eval(zk_ctx* ctx, uint32_t n, const uint64_t* evals, zk_mem evals_mem, const uint64_t* point, uint64_t* out);
/* Range-proof preprocessing of Dag::prove_range, src/dag/mod.rs:1314-1337, one call per auxiliary selection
 * polynomial.  point: the k coordinates of the node's claim; (input_idx[e], table_idx[e]), e < n_sel: the pairs of
 * SelectionPolynomial::selection (util/poly.rs:1017-1022), in idx_mem; the table has 2^table_log entries.
 *   part[t] = sum over the pairs with table_idx = t of eq(point)[input_idx]      (:1324-1329)
 *   middle_claim_out (4 x u64, host) = sum_t part[t] * t                          (:1330)
 *   acc[t] += beta_gamma * part[t]    (:1332-1336 and the fold over the aux polynomials, :1339)
 * acc (2^table_log elements in acc_mem) is updated in place: start from zeros and call once per polynomial.
 * An index >= 2^k or >= 2^table_log is ZK_ERR_ARG (the reference panics on the slice index). */
int zk_range_aux_accumulate(zk_ctx* ctx, uint32_t k, const uint64_t* point, uint64_t n_sel, const uint64_t* input_idx,
                            const uint64_t* table_idx, zk_mem idx_mem, const uint64_t* beta_gamma, uint32_t table_log,
                            uint64_t* acc, zk_mem acc_mem, uint64_t* middle_claim_out);
/* range_dense(n).add_by_scalar(alpha), src/util/poly.rs:1359-1366 and 915-927 (dag/mod.rs:1340): out[i] = i + alpha
 * for i < 2^n (n <= 32: the reference's entries are u32). */
int zk_range_table(zk_ctx* ctx, uint32_t n, const uint64_t* alpha, uint64_t* out, zk_mem out_mem);
/* permute_evals_by_ranges, src/basicblock/einsum.rs:142-198: reorders the variables of a table of 2^n elements
 * of elem_bytes (32: field elements; 16: the i128 witness integers).  ranges holds n_ranges (start, end) pairs
 * of old variable indices; listed one after the other they are the new variable order, lowest first.  Ranges
 * that are invalid, overlap or do not cover all n variables are ZK_ERR_ARG (the reference's asserts).  out
 * must not alias evals. */
int zk_permute_by_ranges(zk_ctx* ctx, uint32_t n, uint32_t elem_bytes, const void* evals, zk_mem evals_mem,
                         uint32_t n_ranges, const uint64_t* ranges, void* out, zk_mem out_mem);
/* fix_variables_zkgpt, src/util/poly.rs:1378-1473: t holds 2^num_vars signed 128-bit little-endian integers
 * (Rust i128), laid out b + c * 2^k; binds the k low variables to point[0..k):
 * out[c] = sum_b eq(point)[b] * t[c * 2^k + b], 2^(num_vars-k) field elements.  The reference's q_bits argument
 * only sizes its table of small multiples and does not change the result; it has no counterpart here. */
int zk_fix_variables_int(zk_ctx* ctx, uint32_t num_vars, const void* t, zk_mem t_mem, uint32_t k, const uint64_t* point,
                         uint64_t* out, zk_mem out_mem);
/* out[lo] = sum_hi weights[hi] * evals[hi * 2^(n-k) + lo]: the contraction inside
 * fix_variables_from_right (poly.rs:719-741) with caller-given weights instead of an eq table
 * (no separate counterpart in the reference; used for trapdoor checksums of commitments). */
int zk_weighted_fold_from_right(zk_ctx* ctx, uint32_t n, const uint64_t* evals, zk_mem evals_mem, uint32_t k,
                                const uint64_t* weights, zk_mem weights_mem, uint64_t* out, zk_mem out_mem);
/* evaluate_lagrange_basis / precompute_eq, src/util/poly.rs:573-618, 657-699: out[x] = eq(x, point)
 * for x < 2^k, variable 0 in index bit 0; k = 0 gives {1}.  point is a host array. */
int zk_eq_table(zk_ctx* ctx, uint32_t k, const uint64_t* point, uint64_t* out, zk_mem out_mem);

/* ---- G1 multi-scalar multiplication ------------------------------------------------------ */
/* P::G1::msm(bases, scalars) of ark-ec's VariableBaseMSM as called at
 * src/crypto/polycommit/kzh2.rs:640 and kzh3.rs:666,772 (and the icicle-feature seam
 * PairingG1::msm, src/crypto/polycommit/mod.rs:72-92): out = sum_i scalars[i] * bases[i].
 * bases: n affine points (64 bytes each); scalars: n Fr elements; out_jac: one Jacobian point
 * (12 x u64).  n = 0 gives the identity (mod.rs:127-130). */
int zk_msm_g1(zk_ctx* ctx, const uint64_t* bases, zk_mem bases_mem, const uint64_t* scalars, zk_mem scalars_mem,
              uint64_t n, uint64_t* out_jac, zk_mem out_mem);
/* The d_x / d_y loops (kzh2.rs:653-660, kzh3.rs:680-687,743-750): n_rows independent MSMs over
 * the same n_bases bases; scalars is row-major n_rows x n_bases; out_jac receives n_rows points. */
int zk_msm_g1_batched(zk_ctx* ctx, const uint64_t* bases, zk_mem bases_mem, uint64_t n_bases, const uint64_t* scalars,
                      zk_mem scalars_mem, uint64_t n_rows, uint64_t* out_jac, zk_mem out_mem);
/* sparse_msm (src/crypto/polycommit/mod.rs:10-31): out = sum_i scalars[i] * all_bases[indices[i]].
 * indices (k x u64) live where the scalars live; an index >= n_bases is ZK_ERR_ARG. */
int zk_msm_g1_gather(zk_ctx* ctx, const uint64_t* all_bases, zk_mem bases_mem, uint64_t n_bases, const uint64_t* indices,
                     const uint64_t* scalars, zk_mem scalars_mem, uint64_t k, uint64_t* out_jac, zk_mem out_mem);
/* CurveGroup::into_affine / normalize_batch for n Jacobian points -> n affine points. */
int zk_g1_normalize(zk_ctx* ctx, const uint64_t* jac, zk_mem jac_mem, uint64_t n, uint64_t* affine_out, zk_mem out_mem);
/* ark-serialize's compressed form of G1 points (what `serialize_compressed` writes: the transcript bytes of a
 * KZH3 commitment, src/crypto/polycommit/kzh3.rs:406-411 through util/serialization.rs:14-21, and the G1 vectors
 * of the SRS files, src/crypto/srs_storage.rs:15-58).  32 bytes per point: x little-endian, bit 7 of the last
 * byte set when y is the larger of {y, q - y}, bit 6 set (and everything else zero) for the point at infinity.
 * Points cross as in the MSM entry points (64 bytes, Montgomery form, infinity = zeros).  Decompression rejects
 * (ZK_ERR_ARG, with the index in zk_last_error) an x >= q, an x with no point above it, and inconsistent flags. */
int zk_g1_compress(zk_ctx* ctx, const uint64_t* affine, zk_mem affine_mem, uint64_t n, uint8_t* out, zk_mem out_mem);
int zk_g1_decompress(zk_ctx* ctx, const uint8_t* in, zk_mem in_mem, uint64_t n, uint64_t* affine_out, zk_mem out_mem);

/* Shape the last MSM on this context chose (window width, windows, largest scalar magnitude in
 * bits, digit entries, buckets): used to report algorithmic work. */
int zk_msm_last_stats(zk_ctx* ctx, int* window_bits, int* windows, int* max_bits, uint64_t* entries, uint64_t* buckets);
/* Work of all the MSMs this context ran since the last reset (a KZH commit runs two, an opening several): the
 * number of MSM pipelines, their non-zero signed digits (each is one mixed addition into a bucket) and the
 * buckets they reduced.  reset != 0 clears the counters after reading.  No counterpart in the reference. */
int zk_msm_work(zk_ctx* ctx, uint64_t* calls, uint64_t* entries, uint64_t* buckets, int reset);

/* ---- KZH2 / KZH3 polynomial commitments, G1 side ------------------------------------------ */
/* Device-resident structured reference string.  dims = 2: KZH2SRS {h_xy, h_y} (kzh2.rs:27-35),
 * split (x_log, y_log) = (n/2, n - n/2) (kzh2.rs:423-429); dims = 3: KZH3SRS {h_xyz, h_yz, h_z}
 * (kzh3.rs:33-45), split as kzh3.rs:429-437.  G2 vectors and pairings stay with the caller. */
typedef struct zk_kzh_srs zk_kzh_srs;
/* setup_kzh2_srs (kzh2.rs:502-555) / setup_kzh3_srs (kzh3.rs:463-563), G1 half, from trapdoors
 * the caller sampled in the reference's order: g (affine), tau_x[2^x_log], tau_y[2^y_log], then
 * alpha (KZH2; tau_z NULL) or tau_z[2^z_log] (KZH3; alpha NULL).  All host arrays. */
int zk_kzh_srs_setup(zk_ctx* ctx, int dims, uint32_t n, const uint64_t* g_affine, const uint64_t* tau_x,
                     const uint64_t* tau_y, const uint64_t* tau_z, const uint64_t* alpha, zk_kzh_srs** out);
/* Sharded SRS: rank `rank` of `world` (a power of two, at most 2^x_log) generates and keeps only
 * its slab of the full vector (whole x-rows); the mid and low vectors are replicated. */
int zk_kzh_srs_setup_sharded(zk_ctx* ctx, int rank, int world, int dims, uint32_t n, const uint64_t* g_affine,
                             const uint64_t* tau_x, const uint64_t* tau_y, const uint64_t* tau_z, const uint64_t* alpha,
                             zk_kzh_srs** out);
/* Commit with a sharded SRS: local_evals = this rank's 2^n / world evaluations (its x-rows).  The
 * partial commitments are summed over ranks and the rows of d_x all-gathered; every rank receives
 * c (8 x u64) and all 2^x_log Jacobian points of d_x. */
int zk_kzh_commit_sharded(zk_ctx* ctx, zk_comm* comm, const zk_kzh_srs* srs, const uint64_t* local_evals,
                          zk_mem evals_mem, uint64_t* c_affine_out, uint64_t* d_x_jac_out);

/* kzh2_open (src/crypto/polycommit/kzh2.rs:676-710) / kzh3_open (kzh3.rs:702-787) over a table sharded by
 * x-rows, the layout of zk_kzh_commit_sharded: local_evals holds this rank's 2^n / world evaluations and srs is
 * the rank's sharded SRS.  d_x_jac (all 2^x_log rows, as zk_kzh_commit_sharded returns them), d_y_jac_out and
 * c_y_affine_out are used for a KZH3 SRS only (NULL otherwise).  Every rank receives the whole opening. */
int zk_kzh_open_sharded(zk_ctx* ctx, zk_comm* comm, const zk_kzh_srs* srs, const uint64_t* local_evals, zk_mem evals_mem,
                        const uint64_t* point, uint32_t point_len, const uint64_t* d_x_jac, uint64_t* d_y_jac_out,
                        uint64_t* c_y_affine_out, uint64_t* f_star_out);
/* An SRS the caller already holds (load_kzh3_srs, src/crypto/srs_storage.rs): h_full 2^n points,
 * h_mid 2^(n - x_log), h_low 2^z_log (KZH3 only). */
int zk_kzh_srs_upload(zk_ctx* ctx, int dims, uint32_t n, const uint64_t* h_full, const uint64_t* h_mid,
                      const uint64_t* h_low, zk_mem mem, zk_kzh_srs** out);
void zk_kzh_srs_free(zk_ctx* ctx, zk_kzh_srs* srs);
int zk_kzh_srs_shape(const zk_kzh_srs* srs, uint32_t* x_log, uint32_t* y_log, uint32_t* z_log);
/* Copy `count` points of vector `which` (0 full, 1 mid, 2 low) from `offset` to a host array. */
int zk_kzh_srs_read(zk_ctx* ctx, const zk_kzh_srs* srs, int which, uint64_t offset, uint64_t count, uint64_t* out);
/* kzh2_commit (kzh2.rs:619-673) / kzh3_commit (kzh3.rs:645-700): evals has 2^poly_n elements,
 * zero-extended to the SRS size.  c_affine_out: 8 x u64; d_x_jac_out: 2^x_log Jacobian points (host). */
int zk_kzh_commit(zk_ctx* ctx, const zk_kzh_srs* srs, uint32_t poly_n, const uint64_t* evals, zk_mem evals_mem,
                  uint64_t* c_affine_out, uint64_t* d_x_jac_out);
/* kzh2_open (kzh2.rs:676-710): f_star_out receives 2^y_log elements (host); the opening's d_x is
 * the commitment's own.  point is padded with leading zeros as split_input does (:479-498). */
int zk_kzh2_open(zk_ctx* ctx, const zk_kzh_srs* srs, uint32_t poly_n, const uint64_t* evals, zk_mem evals_mem,
                 const uint64_t* point, uint32_t point_len, uint64_t* f_star_out);
/* kzh3_open (kzh3.rs:702-787): d_x_jac is the commitment's aux (host, 2^x_log points); outputs
 * (host) d_y_jac_out 2^y_log points, c_y_affine_out 8 x u64, f_star_out 2^z_log elements. */
int zk_kzh3_open(zk_ctx* ctx, const zk_kzh_srs* srs, uint32_t poly_n, const uint64_t* evals, zk_mem evals_mem,
                 const uint64_t* point, uint32_t point_len, const uint64_t* d_x_jac, uint64_t* d_y_jac_out,
                 uint64_t* c_y_affine_out, uint64_t* f_star_out);

/* The G1 and field checks of kzh2_verify (src/crypto/polycommit/kzh2.rs:763-789, steps 2 and 3) and kzh3_verify
 * (kzh3.rs:836-886, checks 2, 4 and 5); the pairing checks (step 1; checks 1 and 3) stay with the caller.
 *   KZH2: MSM(h_y, f_star) == sum_i eq(r_x)[i] d_x[i];  f_star(r_y) == output.
 *   KZH3: c_y == sum_i eq(r_x)[i] d_x[i];  MSM(h_z, f_star) == sum_i eq(r_y)[i] d_y[i];  f_star(r_z) == output.
 * point as for the opens (left-padded to n coordinates); output: 4 x u64; d_x_jac / d_y_jac: Jacobian points as the
 * commit and open return them (d_y_jac and c_y_affine only for a KZH3 SRS, else NULL); f_star: 2^y_log (KZH2) or
 * 2^z_log (KZH3) elements.  All host pointers.  *ok = 1 when every check holds; *failed_check (optional) = the
 * reference's number of the first failing check, 0 when none. */
int zk_kzh_verify_g1(zk_ctx* ctx, const zk_kzh_srs* srs, const uint64_t* point, uint32_t point_len, const uint64_t* output,
                     const uint64_t* d_x_jac, const uint64_t* d_y_jac, const uint64_t* c_y_affine, const uint64_t* f_star,
                     int* ok, int* failed_check);

/* sparse_kzh2_commit (src/crypto/polycommit/sparse_kzh2.rs:14-82) / sparse_kzh3_commit (sparse_kzh3.rs:32-110):
 * the polynomial is given by nnz (index, value) pairs with distinct indices below 2^n (host arrays, in any order).
 * vals may be NULL: every listed entry is then one (a selection polynomial, as the auxiliary polynomials of the
 * lookups are), and the commitment is computed as plain sums of SRS points instead of a multi-scalar product; the
 * same holds for the two opens below. */
int zk_sparse_kzh_commit(zk_ctx* ctx, const zk_kzh_srs* srs, uint64_t nnz, const uint64_t* indices, const uint64_t* vals,
                         uint64_t* c_affine_out, uint64_t* d_x_jac_out);
/* sparse_kzh2_open (sparse_kzh2.rs:84-127): f_star_out receives 2^y_log elements. */
int zk_sparse_kzh2_open(zk_ctx* ctx, const zk_kzh_srs* srs, uint64_t nnz, const uint64_t* indices, const uint64_t* vals,
                        const uint64_t* point, uint32_t point_len, uint64_t* f_star_out);
/* sparse_kzh3_open (sparse_kzh3.rs:112-232); a short point is padded with trailing zeros (:124-131). */
int zk_sparse_kzh3_open(zk_ctx* ctx, const zk_kzh_srs* srs, uint64_t nnz, const uint64_t* indices, const uint64_t* vals,
                        const uint64_t* point, uint32_t point_len, const uint64_t* d_x_jac, uint64_t* d_y_jac_out,
                        uint64_t* c_y_affine_out, uint64_t* f_star_out);

/* Fold for callers that cannot allocate device memory (this entry point has no counterpart in
 * the reference).  Same result as zk_fold_lsb for tables of at most 2^ZK_FOLD_STATIC_MAX_VARS
 * elements; larger n is rejected with ZK_ERR_ARG.  evals_dev and out_dev are device buffers
 * owned by the caller (2^n and 2^(n-k) elements, not overlapping), point is a host array of k
 * elements, stream is the cudaStream_t (or NULL) the work is queued on; the call returns
 * without waiting for it.  It uses the calling thread's current device, takes no zk_ctx, and
 * calls no cudaMalloc / cudaFree or any other allocating routine: the intermediate tables
 * live in a 1.5 MiB array that is part of the library image on every GPU that loads it.
 * The first call on a device looks up that array's device address, and with CUDA's lazy module
 * loading it may also be the moment the driver places the library's code and this array in device
 * memory: make that first call outside any stream capture and before the host hands the rest of
 * HBM to its own pool (a warm-up call on a tiny table is enough).  Later calls on that device
 * leave the free device memory untouched.  All calls on a device share the array (it keeps the previous
 * call's intermediates; nothing in it has to start at zero, every element read was written
 * earlier in the same call), so two calls whose work overlaps on the GPU race: keep them on
 * one stream or order them yourself. */
#define ZK_FOLD_STATIC_MAX_VARS 16
int zk_fold_lsb_static(uint32_t n, const uint64_t* evals_dev, uint32_t k, const uint64_t* point, uint64_t* out_dev,
                       void* stream);

/* ---- seeded synthetic inputs (no counterpart in the reference; its bins draw from StdRng) --- */
/* Element i of stream (seed, stream) = ChaCha20 block `start + i` (key = seed | stream as two
 * little-endian u64 then zeros, zero nonce) read as a 512-bit little-endian integer mod r.
 * Writes `count` elements (Montgomery form) to the device buffer out_dev. */
int zk_gen_uniform_fr(zk_ctx* ctx, uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, uint64_t* out_dev);
/* Same stream; element i = (first keystream word of block start+i, low `bits` bits) - 2^(bits-1),
 * a signed `bits`-bit integer lifted into Fr (negatives as r - |v|), as quantised weights and
 * activations are (src/bin/gpt2.rs:44-49). */
int zk_gen_small_fr(zk_ctx* ctx, uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, int bits,
                    uint64_t* out_dev);

/* Fixed-point activations: element i = round(N(0,1) * 2^scale_log2) (Box-Muller on two keystream
 * words of block start+i, computed in double precision on the device), clamped to +-32767 and
 * lifted into Fr.  Device-generated only: libm on a CPU need not round identically. */
int zk_gen_gauss_fr(zk_ctx* ctx, uint64_t seed, uint64_t stream, uint64_t start, uint64_t count, int scale_log2,
                    uint64_t* out_dev);

/* ---- measurement ---------------------------------------------------------------------- */
/* Throughput probe for the integer roofline (no counterpart in the reference).  kind 0: 32-bit
 * multiply-add, 2 / 3: Montgomery product in Fr / Fq, 4: 32x32+64 multiply-adds inside carry chains (the
 * row primitive of the Montgomery product).  Runs the probe twice and reports the second run: elapsed
 * milliseconds and operations executed. */
int zk_microbench(zk_ctx* ctx, int kind, int blocks, int threads, int iters, float* ms_out, double* ops_out);

#ifdef __cplusplus
}
#endif
#endif /* ZKB200_H */
