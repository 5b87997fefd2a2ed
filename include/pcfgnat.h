/*
 * libpcfgnat — C ABI of the B200 (sm_100a) kernels for PCFG-NAT's structured loss and
 * decoding path.  Plain pointers and sizes only; every pointer is a DEVICE pointer unless
 * marked "host".  The caller owns the memory of inputs, outputs and scratch; the library
 * launches on the stream it is given and never synchronises or calls exit().  It keeps no
 * state between calls, with these exceptions:
 *   - pcfgnat_loss_fwd_bwd_static uses a fixed PCFGNAT_STATIC_SCRATCH_BYTES array inside the
 *     library's device image, shared by all calls on a device (they must not overlap), and
 *     caches that array's address per device (stale after cudaDeviceReset);
 *   - the largest dynamic shared-memory size requested per kernel and device is remembered
 *     (an attribute of the loaded function, also lost by cudaDeviceReset);
 *   - the exchange buffers of pcfgnat_loss_stats_exchange carry an epoch counter from call to call.
 * Each entry point replaces the reference interface cited beside it (paths relative to the
 * reference project root).
 *
 * Conventions shared by all entry points
 *   B            sentences in the batch
 *   L            graph length ("prelen"), padded to the batch maximum
 *   T            target length ("tarlen"), padded to the batch maximum
 *   max_left     links.size(2) - 1 = 2^left_tree_layer - 1; only max_left == 1 is
 *                implemented (every published configuration uses left_tree_layer 1)
 *   Mc, Lt       main-chain / local-tree slots: Mc = (L-2)/(max_left+1)+1, Lt = L-Mc
 *   output_length[b] = m_b graph nodes in use, target_length[b] = n_b target tokens
 *   status       optional device int (may be NULL) the kernels OR PCFGNAT_STATUS_* bits
 *                into; the caller zeroes it and reads it when it wants to
 *   stream       a cudaStream_t passed as void*
 * Return value: PCFGNAT_OK or a negative PCFGNAT_ERR_* code (argument checks and launch
 * errors; asynchronous faults surface on the caller's next synchronisation).
 */
#ifndef PCFGNAT_H_
#define PCFGNAT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PCFGNAT_OK 0
#define PCFGNAT_ERR_INVALID_ARGUMENT (-1) /* null pointer, negative or inconsistent size */
#define PCFGNAT_ERR_UNSUPPORTED (-2)      /* max_left != 1, unsupported dtype */
#define PCFGNAT_ERR_CUDA (-3)             /* a CUDA runtime call or launch failed */
#define PCFGNAT_ERR_WORKSPACE (-4)        /* scratch buffer too small */
#define PCFGNAT_ERR_TOO_LARGE (-5)        /* shape beyond what the kernels index */

/* bits OR-ed into *status by the kernels */
#define PCFGNAT_STATUS_BAD_LENGTH 1 /* a sentence with m_b or n_b out of range was skipped */
#define PCFGNAT_STATUS_BAD_TRACE 2  /* a back-trace left the tables and was cut short */
#define PCFGNAT_STATUS_BAD_INDEX 4  /* a gather index outside [0, V) produced NaN */
#define PCFGNAT_STATUS_TIMEOUT 8    /* a bounded device-side wait ran out */
#define PCFGNAT_STATUS_RECOMPUTED 16 /* pcfgnat_loss_fwd_bwd: a sentence was recomputed in log space (information,
                                        not an error: unusual lengths, or numbers beyond the linear-space range) */

#define PCFGNAT_DTYPE_F32 0
#define PCFGNAT_DTYPE_F16 1

int pcfgnat_version(void);
const char *pcfgnat_error_string(int code);

/* Inside pass.  Replaces pcfg_loss() (fs_plugins/custom_ops/pcfg_loss.cu:379-401, kernels
 * :85-224 and :263-349).  match_all [B][L][T] f32, links [B][L][max_left+1][L] f32,
 * lengths int64.  Writes every cell of S [B][Mc][T+2] and, when C is not NULL, of
 * C [B][Lt][T+2][max_left+2] (fill value -inf); loss_b = S[b][0][0].  S is bit-identical
 * to the reference kernel's table (same reduction order, expf/logf, no fast-math). */
int pcfgnat_loss_fwd(const float *match_all, const float *links, const int64_t *output_length,
                     const int64_t *target_length, int B, int L, int T, int max_left, float *S, float *C,
                     int *status, void *stream);

/* Outside pass + gradients.  Replaces pcfg_loss_backward()
 * (fs_plugins/custom_ops/pcfg_loss_backward.cu:654-721, seven kernels :29-603).
 * grad_output [B] f32, S from pcfgnat_loss_fwd.  S_grad [B][Mc][T+2] is scratch.
 * Writes every cell of match_all_grad [B][L][T] and links_grad [B][L][max_left+1][L]. */
int pcfgnat_loss_bwd(const float *grad_output, const float *S, const float *match_all, const float *links,
                     const int64_t *output_length, const int64_t *target_length, int B, int L, int T, int max_left,
                     float *S_grad, float *match_all_grad, float *links_grad, int *status, void *stream);

/* Forward and backward in one call, as CUDAPCFGLossFunc.forward always runs them
 * (fs_plugins/custom_ops/pcfg_loss.py:63-74).  workspace holds the two DP tables and a small
 * per-sentence record (pcfgnat_loss_workspace_bytes); loss [B] f32 receives S[b][0][0]; gradients
 * are for grad_output == 1.  The tables stay inside the call, so they are built in linear space
 * (probabilities scaled per column: one multiply-add per term instead of one exponential; loss equal
 * to the reference's to ~1e-6 relative, gradients to 1e-3); a sentence whose numbers leave the range
 * of that representation, or whose lengths are unusual, is recomputed in log space within the same
 * call.  PCFGNAT_EXACT_ORDER=1 in the environment keeps everything in the reference's order. */
size_t pcfgnat_loss_workspace_bytes(int B, int L, int T, int max_left);
/* Number of kernels pcfgnat_loss_fwd_bwd / _static launch for this shape on the current device and with the
 * current environment switches: 5 on the linear-space path (inside, outside + gradients, and the three log-space
 * kernels that recompute marked sentences and otherwise return at once); on the log-space path 2 when the outside
 * pass also sums up both gradients, else 3.  For launch accounting; 0 for unsupported arguments. */
int pcfgnat_loss_fwd_bwd_kernels(int B, int L, int T, int max_left);
int pcfgnat_loss_fwd_bwd(const float *match_all, const float *links, const int64_t *output_length,
                         const int64_t *target_length, int B, int L, int T, int max_left, void *workspace,
                         size_t workspace_bytes, float *loss, float *match_all_grad, float *links_grad, int *status,
                         void *stream);

/* The same forward + backward for hosts that cannot hand over scratch memory (a binding that only
 * holds device pointers owned by another framework, or a process whose device memory all belongs
 * to its own arena so that no library may call cudaMalloc).  It has no counterpart in the
 * reference.  The two DP tables live in a fixed PCFGNAT_STATIC_SCRATCH_BYTES array inside the
 * library's device image (held on every GPU that loads the library, until exit); shapes whose
 * pcfgnat_loss_workspace_bytes() exceeds it are refused with PCFGNAT_ERR_TOO_LARGE.  The call
 * allocates nothing.  All calls on a device share the array: calls that may overlap on the GPU
 * race and must be serialised by the caller.  The first call on each device looks up the array's
 * address and should come before any stream capture on that device. */
#define PCFGNAT_STATIC_SCRATCH_BYTES (8u << 20)
int pcfgnat_loss_fwd_bwd_static(const float *match_all, const float *links, const int64_t *output_length,
                                const int64_t *target_length, int B, int L, int T, int max_left, float *loss,
                                float *match_all_grad, float *links_grad, int *status, void *stream);

/* Best tree for glancing training.  Replaces pcfg_best_tree()
 * (fs_plugins/custom_ops/pcfg_best_tree.cu:333-360, kernels :65-197 and :240-301).
 * S from pcfgnat_loss_fwd; tree [B][L] int64: target index emitted by each node, -1 if
 * unused.  Bit-exact with the reference including arg-max tie-breaking. */
int pcfgnat_best_tree(const float *S, const float *match_all, const float *links, const int64_t *output_length,
                      const int64_t *target_length, int B, int L, int T, int max_left, int64_t *tree, int *status,
                      void *stream);

/* Viterbi tables.  Replaces pcfg_viterbi() (fs_plugins/custom_ops/pcfg_viterbi.cu:272-301,
 * kernels :23-140 and :178-241).  ob_lprob [B][L] f32; writes every cell of S f32 and
 * R, Lt, Mt int64, all [B][L][L/4] (fills: -inf, 0).  Bit-exact with the reference. */
int pcfgnat_viterbi(const float *ob_lprob, const float *links, const int64_t *output_length, int B, int L,
                    int max_left, float *S, int64_t *R, int64_t *Lt, int64_t *Mt, int *status, void *stream);

/* Back-trace on the device.  Replaces the host function viterbi_decoding()
 * (fs_plugins/custom_ops/pcfg_loss.cpp:12-73).  Traces [B][L][Q] int64, tokens [B][L]
 * int64, left_tree_mask [mask_dim][mask_dim] int64 (non-zero = not allowed).  Writes
 * out_tokens [B][cap] int64 (pad_index beyond the sentence) and out_count [B] int64. */
int pcfgnat_viterbi_backtrace(const int64_t *pred_length, const int64_t *output_length, const int64_t *Lt,
                              const int64_t *R, const int64_t *Mt, const int64_t *tokens,
                              const int64_t *left_tree_mask, int mask_dim, int64_t pad_index, int B, int L, int Q,
                              int cap, int64_t *out_tokens, int64_t *out_count, int *status, void *stream);

/* Choice of the output length and back-trace in one launch: what the model does between the Viterbi
 * tables and the token list (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:488-502):
 *   scores = S[b][1][len] / penalty[len]  (penalty [Q] f32, the caller's arange(Q) ** beta), NaN -> -inf,
 *   pred_length[b] = first maximum over len = 1 .. Q-1,
 * then the walk of pcfgnat_viterbi_backtrace from that length.  S [B][L][Q] f32 from pcfgnat_viterbi. */
int pcfgnat_viterbi_decode(const float *S, const float *penalty, const int64_t *output_length, const int64_t *Lt,
                           const int64_t *R, const int64_t *Mt, const int64_t *tokens, const int64_t *left_tree_mask,
                           int mask_dim, int64_t pad_index, int B, int L, int Q, int cap, int64_t *pred_length,
                           int64_t *out_tokens, int64_t *out_count, int *status, void *stream);

/* Lookahead / greedy decoding on the device, one launch.  Replaces the decode strategies "lookahead" and "greedy"
 * of the model (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:419-482): the arg-max over
 * (left option, right child) per node of
 *     lookahead != 0:  (links[a][k][c] + ob_lprob[c] * beta) + ob_lprob[left(a, k)] * beta
 *     lookahead == 0:   links[a][k][c]                                  (ob_lprob may be NULL)
 * (first maximum in the order k * L + c), then the reference's in-order walk from node 1 — which it does on the host
 * over links_idx.cpu().tolist() — emitting every visited node's token unless it is pad_index.
 * links [B][L][2][L] f32, ob_lprob [B][L] f32 (max log-prob per node), tokens [B][L] int64, left_tree_mask as for
 * pcfgnat_viterbi_backtrace.  Writes out_tokens [B][cap] int64 (pad_index beyond the sentence) and out_count [B].
 * The reference takes the left-child lookahead term of every sentence from sentence 0 when B > 1
 * (models/...pcfg.py:425); here every sentence uses its own (equal for B == 1, the setting it is published with). */
int pcfgnat_lookahead_decode(const float *links, const float *ob_lprob, const int64_t *tokens,
                             const int64_t *output_length, const int64_t *left_tree_mask, int mask_dim, float beta,
                             int lookahead, int64_t pad_index, int B, int L, int max_left, int cap, int64_t *out_tokens,
                             int64_t *out_count, int *status, void *stream);

/* log-softmax over the vocabulary + gather of selected columns, optional in-place
 * softmax for the backward.  Replaces logsoftmax_gather()
 * (fs_plugins/custom_ops/logsoftmax_gather.cu:295-359, kernel :240-292).
 * logits [rows][V] contiguous, f32 or f16 (PCFGNAT_DTYPE_*); select_idx int64 addressed as
 * select_idx[(r / rows_per_batch) * stride_b + (r % rows_per_batch) * stride_l + s * stride_s]
 * (element strides, so the reference's stride-0 expand of the targets needs no copy);
 * selected [rows][slen] f32.  With require_gradient != 0 the logits are overwritten by
 * the softmax probabilities. */
int pcfgnat_logsoftmax_gather(void *logits, int dtype, const int64_t *select_idx, int64_t stride_b, int64_t stride_l,
                              int64_t stride_s, int64_t rows, int64_t rows_per_batch, int V, int slen,
                              int require_gradient, float *selected, int *status, void *stream);

/* Fused output projection + log-softmax + target gather / row max on the tensor cores; the
 * [rows, V] logits are never written to memory.  New entry point: it stands in for the chain
 * output_projection (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:237, a
 * cuBLAS GEMM inside nn.Linear) -> logsoftmax_gather (fs_plugins/custom_ops/logsoftmax_gather.cu:295-359)
 * on the training / glancing side, and output_projection -> log_softmax(-1).max(-1)
 * (models/...pcfg.py:414-415) on the decoding side.
 * hidden [B*L][H] f16, weight [V][H] f16 (both 16-byte aligned, H a multiple of 64, H <= 512);
 * targets [B][T] int64 or NULL.  Outputs, each optional (NULL = not wanted):
 *   match     [B*L][T] f32  log P(target t | row); with output_length and target_length given
 *                           the criterion's EOS masking is applied
 *                           (fs_plugins/criterions/nat_pcfg_loss.py:112-115)
 * With output_length given (target_length optional) only the rows of real nodes (l < m_b) are
 * projected; the padding rows of every output are set to zero.  Without it all B*L rows are.
 *   max_lprob [B*L]    f32  max_v log P(v | row),   argmax [B*L] int64 its index
 *   lse       [B*L]    f32  log-sum-exp of the row's logits
 * workspace: pcfgnat_proj_workspace_bytes(B, L, T, V) bytes, 16-byte aligned. */
size_t pcfgnat_proj_workspace_bytes(int B, int L, int T, int V);
int pcfgnat_proj_logsoftmax_gather(const void *hidden, const void *weight, const int64_t *targets,
                                   const int64_t *output_length, const int64_t *target_length, int B, int L, int T,
                                   int V, int H, float *match, float *max_lprob, int64_t *argmax, float *lse,
                                   void *workspace, size_t workspace_bytes, int *status, void *stream);

/* Backward of pcfgnat_proj_logsoftmax_gather with respect to the logits, without the [rows][V] log-probabilities
 * ever having been stored: the logits tiles are recomputed on the tensor cores and turned into
 *   dlogits[row][v] = sum_t grad_match[row][t] * ([targets[t] == v] - exp(logit[row][v] - lse[row]))
 * written as bf16 [B*L][V] (16-byte aligned; rows of padding nodes, l >= m_b, are zero).  It stands in for the
 * in-place softmax buffer of logsoftmax_gather (fs_plugins/custom_ops/logsoftmax_gather.cu:278-289) and the
 * backward of DagLogsoftmaxGatherFunc (fs_plugins/custom_ops/pcfg_loss.py:168-180); the caller finishes with two
 * plain GEMMs: d hidden = dlogits . weight, d weight = dlogits^T . hidden.  lse [B*L] f32 is the forward's
 * output; grad_match [B*L][T] f32; entries the forward masked as EOS (both lengths given) get no gradient.
 * workspace: pcfgnat_proj_workspace_bytes(B, L, T, V) bytes. */
int pcfgnat_proj_dlogits(const void *hidden, const void *weight, const int64_t *targets, const int64_t *output_length,
                         const int64_t *target_length, const float *lse, const float *grad_match, int B, int L, int T, int V,
                         int H, void *dlogits, void *workspace, size_t workspace_bytes, int *status, void *stream);

/* pcfgnat_proj_dlogits for the real graph nodes only: row i of dlogits [capacity][V] belongs to the i-th real node of
 * the batch (sentence after sentence, nodes l < m_b), so that the caller's two GEMMs run over sum_b m_b rows
 * instead of B*L.  row_index [capacity] i64 receives the padded position b * L + l of every compact row (0 beyond
 * the last one) for the gather of the states and the scatter of their gradient, n_rows (device, may be null) their
 * number.  capacity is normally sum_b m_b as the host knows it (at most B*L); a batch with more real nodes than
 * capacity sets PCFGNAT_STATUS_BAD_LENGTH and writes only the first capacity rows. */
int pcfgnat_proj_dlogits_compact(const void *hidden, const void *weight, const int64_t *targets,
                                 const int64_t *output_length, const int64_t *target_length, const float *lse,
                                 const float *grad_match, int B, int L, int T, int V, int H, int capacity, void *dlogits,
                                 int64_t *row_index, int *n_rows, void *workspace, size_t workspace_bytes, int *status,
                                 void *stream);

/* The two matrix products that finish the backward of the projection, on the tcgen05 tensor cores (bf16 operands,
 * float32 accumulation), in place of autograd's GEMMs of nn.Linear behind DagLogsoftmaxGatherFunc.backward
 * (fs_plugins/custom_ops/pcfg_loss.py:168-180, models/glat_decomposed_with_link_two_hands_tri_pcfg.py:237):
 *   d_rows   [n][H] f32 = dlogits [n][V] . weight_bf16 [V][H]
 *   d_weight [V][H] f32 = dlogits^T . rows_bf16 [n][H]
 * dlogits [n][V] bf16 as pcfgnat_proj_dlogits(_compact) writes it, rows_bf16 the decoder states of the same n rows.
 * Either output may be NULL (that product is skipped).  V and H must be multiples of 8 and all pointers 16-byte
 * aligned (PCFGNAT_ERR_UNSUPPORTED / _INVALID_ARGUMENT otherwise); n is a host value, so the call cannot be part
 * of a captured graph that is replayed for batches with other row counts. */
int pcfgnat_proj_backward_gemms(const void *dlogits, const void *weight_bf16, const void *rows_bf16, int n, int V, int H,
                                float *d_rows, float *d_weight, int *status, void *stream);

/* The three numbers the criterion's scalar loss is formed from, in one launch
 * (fs_plugins/criterions/nat_pcfg_loss.py:117-135: sentences whose loss is infinite or NaN are
 * counted and left out, the others are divided by their target length):
 *   stats[0] = sum_b loss[b] / max(target_length[b], 1) over valid sentences,
 *   stats[1] = B,   stats[2] = number of invalid sentences.
 * The caller sums stats over ranks and forms -stats[0] / stats[1]. */
int pcfgnat_loss_stats(const float *sentence_loss, const int64_t *target_length, int B, float *stats, void *stream);

/* pcfgnat_loss_stats summed over the `world` GPUs of a sentence-sharded job in the same launch: each rank
 * stores its three numbers into every peer's exchange buffer (plain peer stores over NVLink) and adds, in rank
 * order, what the peers stored into its own; stats [3] is then the same on every rank.  It stands in for the
 * all-reduce of the criterion's logging outputs that fairseq's trainer issues after every update.
 * peer_buffers: device array of `world` device pointers, entry r = rank r's exchange buffer as mapped in THIS
 * process (peer-accessible memory, e.g. torch symmetric memory), each PCFGNAT_EXCHANGE_BYTES(world) bytes,
 * zero-filled before the first call and used for nothing else.  Every rank must make the same sequence of
 * calls.  The wait for a peer is bounded (2^21 polls 200 ns apart: about half a second).  When a peer has not
 * arrived by then the call does NOT return a short sum: all three numbers of `stats` are NaN on the rank that
 * gave up and PCFGNAT_STATUS_TIMEOUT is set in `status`; the context stays usable.  A caller whose ranks may
 * drift further apart than that (a checkpoint written by one rank, validation on rank 0) must either line the
 * ranks up before the step or sum pcfgnat_loss_stats with an all-reduce, which simply waits. */
#define PCFGNAT_EXCHANGE_MAX_WORLD 32
#define PCFGNAT_EXCHANGE_BYTES(world) (64u + 64u * (unsigned)(world))
int pcfgnat_loss_stats_exchange(const float *sentence_loss, const int64_t *target_length, int B,
                                const uint64_t *peer_buffers, int rank, int world, float *stats, int *status,
                                void *stream);

/* Glancing sampler between the two decoder passes (fs_plugins/criterions/nat_pcfg_loss.py:216-267), one launch
 * instead of ~15 torch operators.
 * path [B][L] int64: aligned target position of each graph node (the best tree), negative = none;
 * pred_tokens [B][L], tgt_tokens [B][T], prev_output_tokens [B][L] int64.  The random draws are the caller's
 * (torch's generator stays the source of randomness): noise [B][L] f32 standard-normal (the reference's
 * torch.randn; strategies NUMBER_RANDOM and CMLM), uniform f32 in [0, 1) (the reference's torch.rand): [B] for
 * CMLM, [B][L] for FRACTION, unused (may be NULL) for NUMBER_RANDOM.  strategy = the criterion's
 * --glance-strategy: "number-random", "cmlm", or none (FRACTION).  Outputs:
 *   matchmask [B][T][L] u8   1 where node l is aligned to target t
 *   oracle    [B][L]   int64 target token of the node's alignment (position 0 when unaligned)
 *   same_num  [B]      int64 aligned nodes whose predicted token already equals the oracle
 *   glance_num[B]      int64 NUMBER_RANDOM: (long)((n_b - same_num) * context_p + 0.5) in float32;
 *                            CMLM: (long)(n_b * uniform[b] + 0.5); FRACTION: the number of kept nodes
 *   keep      [B][L]   u8    NUMBER_RANDOM / CMLM: the glance_num nodes with the largest noise among the aligned
 *                            ones (ties and glance_num beyond the aligned count as torch.sort + >= give);
 *                            FRACTION: aligned and uniform[b][l] < (n_b - same_num) / n_b * context_p
 *   glat_prev [B][L]   int64 prev_output_tokens with the oracle token at the kept nodes
 * For the two counting strategies the reference's second draw (rand < keep_prob, keep_prob in {0,1}) selects the
 * same mask. */
#define PCFGNAT_GLANCE_NUMBER_RANDOM 0
#define PCFGNAT_GLANCE_CMLM 1
#define PCFGNAT_GLANCE_FRACTION 2
int pcfgnat_glance_select(const int64_t *path, const int64_t *pred_tokens, const int64_t *tgt_tokens,
                          const int64_t *prev_output_tokens, const int64_t *target_length, const float *noise,
                          const float *uniform, int strategy, float context_p, int B, int L, int T, uint8_t *matchmask,
                          int64_t *oracle, int64_t *same_num, int64_t *glance_num, uint8_t *keep, int64_t *glat_prev,
                          void *stream);

/* Force-emit mask of the training pass (fs_plugins/criterions/nat_pcfg_loss.py:116-121, active unless
 * --no-force-emit): a node whose token the glancing sampler revealed (keep [B][L] u8) may only emit the target
 * position it is aligned to (matchmask [B][T][L] u8, as pcfgnat_glance_select writes it):
 *   out[b][l][t] = keep[b][l] && !matchmask[b][t][l] ? -inf : match[b][l][t]
 * and, as the reference detaches that part, carries no gradient:
 *   out[b][l][t] = keep[b][l] ? 0 : grad[b][l][t]            (pcfgnat_force_emit_grad)
 * match, grad, out [B][L][T] f32; out may be the input itself. */
int pcfgnat_force_emit(const float *match, const uint8_t *matchmask, const uint8_t *keep, int B, int L, int T,
                       float *out, void *stream);
int pcfgnat_force_emit_grad(const float *grad, const uint8_t *keep, int B, int L, int T, float *out, void *stream);

/* The transition log-probabilities links [B][L][2][L] f32 from the projected link features: extract_links()
 * after its link projections (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:163-199) as
 * three launches.  Only main-chain nodes have, or are, right children, so everything is
 * compact over the M main-chain nodes: nodes [M] int32 = their ids (ascending), slot_of [L] int32 = index of a
 * node among them or -1.
 *  1. pcfgnat_links_gather_features: q, kl, kr [B][L][heads][head_dim] (dtype PCFGNAT_DTYPE_F16 or PCFGNAT_DTYPE_F32) ->
 *     float32 GEMM operands qm = q[nodes], krm = kr[nodes] ([B][heads][M][head_dim]) and klm
 *     ([B][heads][M+1][head_dim]: row 0 = kl[0], "no left child"; row 1 + s = kl[nodes[s] - 1]);
 *  2. pcfgnat_links_scores: ac [B][heads][M][M] = qm krm^T, bc [B][heads][M+1][M] = klm krm^T, unscaled (small
 *     batched float32 products);
 *  3. pcfgnat_links_from_scores: masking of inadmissible children, the two left options (none, node a-1), the
 *     joint log-softmax over (left option, right child) per head with scores scaled by 1/sqrt(head_dim), the
 *     log-sum-exp mixture of the heads with log-softmax(gate_logits [B][L][heads]), -inf rows for nodes without an
 *     admissible left or right child.  nonpad [B][L] u8 (token != pad); left_tree_mask, right_tree_mask [L][L] u8
 *     (1 = not allowed) and main_chain [L] u8 as lemon_tree.get_mask gives them. */
int pcfgnat_links_gather_features(const void *q, const void *kl, const void *kr, int dtype, const int *nodes, int M,
                                  int B, int L, int heads, int head_dim, float *qm, float *klm, float *krm, void *stream);
int pcfgnat_links_scores(const float *qm, const float *klm, const float *krm, int M, int B, int heads, int head_dim,
                         float *ac, float *bc, void *stream);
/* Gradient of those links with respect to the link features and the gate logits (training; the reference gets it
 * from autograd through the ~30 operators of extract_links).  links_grad [B][L][2][L] f32; ac, bc, qm, klm, krm and
 * the masks as in the forward.  Scratch: X0, X1 [B][heads][M][M] and dab [B][heads][M][2] f32 (fully overwritten at
 * the rows of main-chain nodes; the caller zero-fills them once for the others).  Outputs, all f32: dq, dkl, dkr
 * [B][L][heads][head_dim] (zero-filled by the caller: only main-chain nodes and their left options are written)
 * and dgates [B][L][heads] (every cell written). */
int pcfgnat_links_backward(const float *links_grad, const float *ac, const float *bc, const float *qm, const float *klm,
                           const float *krm, const float *gate_logits, const uint8_t *nonpad,
                           const uint8_t *left_tree_mask, const uint8_t *right_tree_mask, const uint8_t *main_chain,
                           const int *slot_of, const int *nodes, int M, int B, int L, int heads, int head_dim, int max_left,
                           float *X0, float *X1, float *dab, float *dq, float *dkl, float *dkr, float *dgates,
                           void *stream);
int pcfgnat_links_from_scores(const float *ac, const float *bc, const float *qm, const float *klm,
                              const float *gate_logits, const uint8_t *nonpad, const uint8_t *left_tree_mask,
                              const uint8_t *right_tree_mask, const uint8_t *main_chain, const int *slot_of,
                              const int *nodes, int M, int B, int L, int heads, int head_dim, int max_left, float *links,
                              void *stream);

/* Copies the rows of a transition tensor that the kernels read — links[b][a][.][.] for main-chain nodes a
 * (odd a at max_left == 1) — from src to dst, both [B][L][max_left+1][L] f32, either of them in host
 * (preferably pinned) or device memory; asynchronous on `stream` (one strided cudaMemcpy2DAsync).  The other
 * rows of dst are left as they are: a staging buffer filled with -inf once stays valid.  Host plumbing for
 * callers that stage batches from host memory: it halves the bytes the largest input sends over PCIe. */
int pcfgnat_copy_links_main_rows(void *dst, const void *src, int B, int L, int max_left, void *stream);

/* Copies the rows of the real graph nodes of sentences [b0, b1) from src to dst, both [B][L][row_bytes]:
 * rows l < m_b with m_b = host_lengths[b] clamped to [0, L]; one cudaMemcpyAsync per run of adjacent rows on
 * `stream`, through the copy engine, no kernel.  A copy costs the host several microseconds, so with max_copies > 0
 * at most that many are issued: runs are joined across the smallest gaps of padding rows, which are then sent along
 * (0 = one copy per sentence, or per group of sentences that fill their L rows).  rows_sent (host, may be NULL)
 * receives the number of rows copied.  host_lengths [B] int64 is a HOST array, read before the call returns.  Padding rows of dst that are not sent keep what they held (no kernel of
 * this library reads them).  Host plumbing with no counterpart in the reference, whose inputs are made on the
 * device: for a training batch it sends 11 to 13 MB of decoder states where the padded tensor has 15 MB. */
int pcfgnat_copy_real_rows(void *dst, const void *src, const int64_t *host_lengths, int b0, int b1, int L,
                           size_t row_bytes, int max_copies, int64_t *rows_sent, void *stream);

/* The copies pcfgnat_copy_real_rows would issue for the same arguments, without issuing them (host arithmetic only, no
 * CUDA call): runs [2 * i] = first row and runs [2 * i + 1] = number of rows of copy i, in rows of the [B * L] view.
 * Returns the number of copies (at most min(b1 - b0, max_copies if > 0)), or a negative error when `capacity` pairs
 * do not hold them.  For callers that size pinned staging or account for the bytes beforehand, and for tests. */
int pcfgnat_plan_real_rows(const int64_t *host_lengths, int b0, int b1, int L, int max_copies, int64_t *runs,
                           int capacity);

/* Fetches a batch's large inputs from HOST memory with one kernel that reads the host buffers itself (mapped pinned
 * memory, e.g. cudaHostAlloc / torch pin_memory; device memory works too), and only what the kernels of this library
 * read: the decoder states of the real graph nodes, hidden[b][l][.] for l < m_b (row_bytes per node, a multiple of
 * 16), and the transitions links[b][a][k][c] for main-chain a < m_b and a < c < m_b; the other cells of the
 * main-chain rows of links_dst are set to -inf, rows of other nodes are left as they are (fill the buffer with -inf
 * once).  Either pair of pointers may be NULL.  output_length [B] int64 is a DEVICE array and must be there when the
 * kernel runs.  Host plumbing with no counterpart in the reference, whose inputs are made on the device: for a
 * training batch it moves about 14 MB over PCIe where the padded tensors have 33 MB.  The host buffers must not
 * change until the kernel has run. */
int pcfgnat_stage_inputs(const void *hidden_src, void *hidden_dst, int row_bytes, const float *links_src,
                         float *links_dst, const int64_t *output_length, int B, int L, int max_left, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PCFGNAT_H_ */
