/*
 * flare_b200 -- C ABI of the sm_100a FLARE gather-scatter token mixer.
 *
 * The reference project (vpuri3/FLARE.py) has no native interface: its hot
 * path is two adjacent calls of torch's scaled_dot_product_attention inside
 * Python modules.  The entry points below are what a binding for that path
 * calls instead; every one cites the reference lines it replaces.
 *
 *   S = scale * q k^T            (M x N per (b,h); never materialised)
 *   gather :  z = softmax_N(S) v           L_m = logsumexp_n S_mn
 *   scatter:  y = softmax_M(S^T) z         C_n = logsumexp_m S_mn
 *
 * Conventions
 *   - Plain pointers and sizes only.  All pointers are DEVICE pointers unless
 *     a comment says otherwise.  The library never allocates, frees or keeps
 *     device memory: the caller passes every output and the workspace.
 *   - Token tensors k, v, y, dy, dk, dv are [B,H,N,D] with arbitrary element
 *     strides for b, h, n and unit stride for d (the 'b n (h d) -> b h n d'
 *     views of pdebench/models/flare.py:127-128 are passed as they are).
 *     q is [H,M,D] (q_stride[0] == 0, shared by the batch, flare.py:126,136)
 *     or [B,H,M,D].  Base pointers and row pitches must be 16-byte aligned.
 *   - z32, dz32 are contiguous fp32 [B,H,M,D]; lse_m is fp32 [B,H,M]; lse_n and
 *     delta_n are fp32 [B,H,N]; natural-log units.
 *   - A partial record is fp32 [parts][B][H][M][D+2]: columns 0..D-1 hold
 *     sum_n exp(S_mn - m) v_n, column D the running maximum m, column D+1 the
 *     sum of exp(S_mn - m).  Token ranges on one GPU and the shards of a
 *     context-parallel group use the same record and the same combine.
 *   - key_mask is uint8 [B,N] (contiguous), non-zero = keep; NULL = keep all
 *     (lra/models/backends.py:615-622).
 *   - Every call is asynchronous on `stream`, never synchronises the host, may
 *     be made from several host threads and on several devices of one process
 *     (per-device state is set up once, under a lock), and returns 0 when the
 *     work was enqueued, or a negative FLARE_E* code when the request was
 *     rejected before any launch; flare_last_error() then describes why.
 *     flare_gather_noalloc is the exception to re-entrancy: see there.
 */
#ifndef FLARE_B200_H_
#define FLARE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLARE_F32  0
#define FLARE_F16  1
#define FLARE_BF16 2

#define FLARE_OK             0
#define FLARE_EINVAL        -1   /* bad shape / dtype / null pointer            */
#define FLARE_EALIGN        -2   /* pointer or stride not 16-byte aligned       */
#define FLARE_EWORKSPACE    -3   /* workspace too small                         */
#define FLARE_ECUDA         -4   /* a CUDA runtime call failed                  */
#define FLARE_EUNSUPPORTED  -5   /* shape outside what the kernels cover        */

/* which softmax terms a backward call differentiates */
#define FLARE_TERM_GATHER   1    /* dS1 = P (dZ V^T - Delta)                    */
#define FLARE_TERM_SCATTER  2    /* dS2 = A (Z dY^T - delta)                    */
#define FLARE_TERM_BOTH     3

/* flare_set_path: a testing aid, not a second implementation.  The tensor-core kernels serve bf16 and
 * fp16 with D in {16,32} (bf16 D = 64 in the forward passes); the fp32-arithmetic kernels serve fp32
 * and every other shape.  SIMT forces the latter for 16-bit inputs too, TC_EXACT keeps the tensor-core
 * kernels but always takes the general two-exponential backward. */
#define FLARE_PATH_AUTO     0
#define FLARE_PATH_SIMT     1
#define FLARE_PATH_TC_EXACT 2

typedef void* flare_stream_t;    /* a cudaStream_t */

typedef struct FlareProblem {
  int32_t B, H, N, M, D;
  int32_t dtype;                 /* FLARE_F32 | FLARE_F16 | FLARE_BF16: q,k,v,y,dy,dk,dv */
  float   scale;                 /* attn_scale of the reference (1.0 or D^-0.5)          */
  int32_t n_splits;              /* token ranges per (b,h) in the split passes; 0 = auto  */
  int64_t q_stride[3];           /* b (0 = shared latents), h, m                          */
  int64_t k_stride[3];           /* b, h, n  (elements)                                   */
  int64_t v_stride[3];
  int64_t y_stride[3];
  int64_t dy_stride[3];
  int64_t dk_stride[3];
  int64_t dv_stride[3];
  /* Attention dropout of both SDPA calls (dropout_p of lra/models/backends.py:604-606): every softmax
   * weight is zeroed with probability dropout_p and the survivors are scaled by 1/(1-dropout_p), after
   * the normalisation, independently in the gather (weights P) and in the scatter (weights A).  The
   * keep decision of element (call, b, h, m, n) is a hash of those indices and dropout_seed, so the
   * backward passes regenerate the masks of the forward from the same two numbers.  0 = off.  Served by
   * the tensor-core kernels only (16-bit dtype, D in {16,32}); refused with FLARE_EUNSUPPORTED elsewhere. */
  float    dropout_p;
  uint64_t dropout_seed;
} FlareProblem;

int         flare_version(void);
const char* flare_last_error(void);          /* host string, thread-local */
int         flare_set_path(int path);        /* returns the previous setting */

/* Number of token ranges the split passes use for this problem (>= 1). */
int    flare_pick_splits(const FlareProblem* p);
/* Bytes of scratch the two whole-pass calls need (upper bounds, 256-byte aligned sizes). */
size_t flare_fwd_workspace_bytes(const FlareProblem* p);
size_t flare_bwd_workspace_bytes(const FlareProblem* p);

/* ---- whole passes on one GPU ------------------------------------------------
 * flare_mixer_fwd replaces the two SDPA calls of README.md:49-50 /
 * pdebench/models/flare.py:137-138 / lra/models/backends.py:605-606:
 * y = SDPA(k, q, SDPA(q, k, v)).  It also returns what the backward needs.   */
int flare_mixer_fwd(const FlareProblem* p, const void* q, const void* k, const void* v,
                    const uint8_t* key_mask, void* y, float* z32, float* lse_m, float* lse_n,
                    void* workspace, size_t workspace_bytes, flare_stream_t stream);

/* flare_mixer_bwd replaces autograd through those two SDPA calls (the reference
 * has no hand-written backward; torch's SDPA backward plus the reduction that
 * expand() of flare.py:136 adds).  dq32 is fp32 [H,M,D] (summed over the batch)
 * when q_stride[0] == 0, else fp32 [B,H,M,D].                                  */
int flare_mixer_bwd(const FlareProblem* p, const void* q, const void* k, const void* v,
                    const void* dy, const void* y, const uint8_t* key_mask,
                    const float* z32, const float* lse_m, const float* lse_n,
                    float* dq32, void* dk, void* dv,
                    void* workspace, size_t workspace_bytes, flare_stream_t stream);

/* ---- the passes one by one (context-parallel callers put a collective between
 * them; BigFLARE of pdebench/models/flare_ablations.py:93-132 modifies z between
 * gather and scatter) --------------------------------------------------------- */

/* First SDPA call, per token range: rec[S][B][H][M][D+2], S = p->n_splits (must be >= 1). */
int flare_gather_partial(const FlareProblem* p, const void* q, const void* k, const void* v,
                         const uint8_t* key_mask, float* rec, flare_stream_t stream);

/* Log-sum-exp combine of n_parts records.  Any of z32, z_out (p->dtype, [B,H,M,D]
 * contiguous), lse_m, rec_out (one merged, un-normalised record) may be NULL. */
int flare_combine(const FlareProblem* p, const float* rec, int n_parts, float* z32,
                  void* z_out, float* lse_m, float* rec_out, flare_stream_t stream);

/* flare_combine / flare_reduce_sum over one buffer per rank instead of one strided array: `rec_ptrs` /
 * `part_ptrs` is a DEVICE array of n_parts device pointers, each to a [B,H,M,D+2] record (resp. a
 * rows x width array), on this GPU or in a peer GPU's memory mapped into this process (symmetric
 * memory, IPC); the kernels read them with plain loads over NVLink, in index order on every rank, so
 * all ranks get bit-identical results.  This is the context-parallel all-gather (resp. all-reduce)
 * fused into its consumer; the caller orders it after the peers' writes (a barrier on the stream).
 * No counterpart in the reference (its only parallelism is data-parallel replicas). */
int flare_combine_peers(const FlareProblem* p, const float* const* rec_ptrs, int n_parts, float* z32,
                        void* z_out, float* lse_m, float* rec_out, flare_stream_t stream);
int flare_reduce_sum_peers(const float* const* part_ptrs, int n_parts, int64_t rows, int width,
                           float* out, flare_stream_t stream);

/* A context-parallel group on one node as the kernels see it.  Every rank owns an exchange buffer and an
 * int32[world] array of arrival flags (zero before the first exchange) in memory its peers have mapped.
 * An exchange: write this rank's contribution into `mine`, flare_peer_barrier, read all of `bufs` in the
 * consuming kernel.  `epoch` numbers the exchanges of the group: the same on all ranks for one exchange,
 * larger for every later one; a buffer may be rewritten two exchanges later (use two alternately).
 * The barrier's wait is bounded (about half a second): on expiry bit 1 of the device status word is set
 * and the step's result is invalid, but nothing hangs.  Each rank must run on its own GPU.
 * No counterpart in the reference. */
typedef struct FlarePeers {
  int32_t rank, world;
  const float* const* bufs;    /* DEVICE array [world] of device pointers: each rank's exchange buffer */
  float* mine;                 /* this rank's exchange buffer (the memory bufs[rank] points to)          */
  int32_t* const* flags;       /* DEVICE array [world] of device pointers: each rank's flag array,
                                  int32[world + 1], zero before the first exchange                        */
  int32_t epoch;               /* number of this exchange: 1, 2, 3 ... alike on every rank; or 0 on every
                                  exchange: the barrier then counts for itself in flags[rank][world], and a
                                  recorded launch sequence (a CUDA graph) can be replayed unchanged        */
} FlarePeers;
int flare_peer_barrier(const FlarePeers* g, flare_stream_t stream);

/* flare_mixer_fwd / flare_mixer_bwd over a token axis sharded across the group: k, v, y, dy, dk, dv are this
 * rank's shard, z32 / lse_m come out identical on every rank.  The exchanges are the merged gather record
 * (B*H*M*(D+2) floats), dZ (B*H*M*D) and, unless `dq` is NULL, dQ (the size of dq32); each FlarePeers
 * names buffers of at least that size.  Workspaces as for the single-GPU calls. */
int flare_cp_mixer_fwd(const FlareProblem* p, const void* q, const void* k, const void* v,
                       const uint8_t* key_mask, void* y, float* z32, float* lse_m, float* lse_n,
                       void* workspace, size_t workspace_bytes, const FlarePeers* rec, flare_stream_t stream);
int flare_cp_mixer_bwd(const FlareProblem* p, const void* q, const void* k, const void* v, const void* dy,
                       const void* y, const uint8_t* key_mask, const float* z32, const float* lse_m,
                       const float* lse_n, float* dq32, void* dk, void* dv, void* workspace,
                       size_t workspace_bytes, const FlarePeers* dz, const FlarePeers* dq, flare_stream_t stream);

/* Second SDPA call: y = softmax_M(k q^T) z32; lse_n may be NULL. */
int flare_scatter(const FlareProblem* p, const void* q, const void* k, const float* z32,
                  const uint8_t* key_mask, void* y, float* lse_n, flare_stream_t stream);

/* dZ = A dY per token range: dz_part[S][B][H][M][D] fp32. */
int flare_bwd_dz_partial(const FlareProblem* p, const void* q, const void* k, const void* dy,
                         const uint8_t* key_mask, const float* lse_n, float* dz_part,
                         flare_stream_t stream);

/* out[rows][width] = sum over n_parts of parts[part][rows][width] (ordered, deterministic). */
int flare_reduce_sum(const float* parts, int n_parts, int64_t rows, int width, float* out,
                     flare_stream_t stream);

/* Per-token gradients dk, dv and delta_n = dy_n . y_n.  `terms` selects which
 * softmax is differentiated; v / dz32 / lse_m may be NULL without FLARE_TERM_GATHER,
 * dy / y / lse_n without FLARE_TERM_SCATTER (then dk only gets the gather term). */
int flare_bwd_tokens(const FlareProblem* p, int terms, const void* q, const void* k, const void* v,
                     const void* dy, const void* y, const uint8_t* key_mask,
                     const float* z32, const float* dz32, const float* lse_m, const float* lse_n,
                     void* dk, void* dv, float* delta_n, flare_stream_t stream);

/* dQ per token range: dq_part[S][B][H][M][D] fp32 (reduce with flare_reduce_sum). */
int flare_bwd_dq_partial(const FlareProblem* p, int terms, const void* q, const void* k,
                         const void* v, const void* dy, const uint8_t* key_mask,
                         const float* z32, const float* dz32, const float* lse_m,
                         const float* lse_n, const float* delta_n, float* dq_part,
                         flare_stream_t stream);

/* flare_bwd_tokens and flare_bwd_dq_partial in one call: dk, dv and dq_part[S][B][H][M][D] from a
 * single sweep over k, v, dy, y where a fused tensor-core kernel covers the problem (bf16 or fp16,
 * D in {16,32}, up to 1024 latents; key_mask and single terms included), else the two launches above.
 * delta_n [B,H,N] fp32 (256-byte aligned) is scratch; it may be left unwritten.  `terms` and the
 * pointers that may be NULL are as for flare_bwd_tokens.  Stream-ordered: no host synchronisation.
 * Replaces the bulk of autograd through the two SDPA calls of pdebench/models/flare.py:137-138. */
int flare_bwd_main(const FlareProblem* p, int terms, const void* q, const void* k, const void* v,
                   const void* dy, const void* y, const uint8_t* key_mask, const float* z32,
                   const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                   float* delta_n, float* dq_part, flare_stream_t stream);

/* Gather (first SDPA call) that allocates nothing and needs no workspace.  It has no counterpart
 * in the reference.  It exists for callers that may not allocate device memory at the point of
 * the call: plugins running inside a host framework's fixed memory plan, latency-critical service
 * threads that must stay out of the allocator, callers that own nothing but the tensors passed in.
 * The split-N partial records go to a FLARE_NOALLOC_SCRATCH_BYTES array built into the library
 * (resident on every GPU that loads it, until exit).  Refused with FLARE_EWORKSPACE when one record
 * set, B*H*M*(D+2) floats, does not fit; with fewer token ranges than usual when only those fit.
 * Outputs as flare_combine: z32 fp32 [B,H,M,D], z_out in p->dtype, lse_m fp32 [B,H,M]; any may be
 * NULL but not all.  All calls share the array: calls that overlap on the GPU (other streams,
 * other host threads) race and must be serialised by the caller.  The first call on a device
 * resolves the array's device address and should be made outside any stream capture; like every call
 * of this entry point it must not run concurrently with another one. */
#define FLARE_NOALLOC_SCRATCH_BYTES (16u << 20)
int flare_gather_noalloc(const FlareProblem* p, const void* q, const void* k, const void* v,
                         const uint8_t* key_mask, float* z32, void* z_out, float* lse_m,
                         flare_stream_t stream);

/* Causal FLARE: y_t = softmax_M(S[:,t]) . z_t with z_t = softmax_{n<=t}(S) v.  The reference links
 * this path (README.md:60) but ships no code, formula or test vector for it (figs/flare_decoder.py only
 * animates a diagram): the definition -- token t sees tokens 0..t inclusive -- is this library's choice,
 * checked for self-consistency only (dense == recurrent == chunked forms; prefill == token-by-token decode).
 * The state is one gather record per (b, h): float [B,H,M,D+2] = (acc[D], m, l) per latent, the same
 * record flare_gather_partial writes; start from acc = 0, m = -inf, l = 0.
 *   flare_causal_prefill: all N tokens at once.  workspace: flare_causal_workspace_bytes(p) bytes.
 *     state_in (may be NULL: empty prefix) is the record before token 0, state_out (may be NULL)
 *     receives the record after token N-1.
 *   flare_causal_decode: the N tokens of k, v (usually N = 1) one after the other on `state`,
 *     updated in place.
 * Requires D in {16,32,64,128}, M a multiple of 256/D and at most 32*256/D; dtype as p->dtype.
 * bf16 with M <= 128, D in {32,64} and 16-byte aligned rows runs the prefill's chunk records and chunk
 * walk on the tensor cores (five tcgen05 products per 128-token chunk); a chunk whose scores climb by
 * more than 64 octaves is redone, inside the same call, by the fp32 walk.  On that path the chunk records
 * travel between the passes as 16-bit acc rows (summed in fp32), so state_out carries bf16 rounding of the
 * chunk sums; `workspace` must be 16-byte aligned. */
size_t flare_causal_workspace_bytes(const FlareProblem* p);
int flare_causal_prefill(const FlareProblem* p, const void* q, const void* k, const void* v, void* y,
                         const float* state_in, float* state_out, float* workspace,
                         flare_stream_t stream);
int flare_causal_decode(const FlareProblem* p, const void* q, const void* k, const void* v, void* y,
                        float* state, flare_stream_t stream);

/* Backward of flare_causal_prefill from an empty prefix: dq32 [B][H][M][D] fp32 (one latent gradient per
 * (b, h): sum over b when the latents are shared), dk, dv with dk_stride / dv_stride, from dy (dy_stride).
 * A reverse scan over 128-token chunks on the forward's own chunk-start records, which it rebuilds in
 * `workspace` (flare_causal_bwd_workspace_bytes(p) bytes); fp32 arithmetic.  D in {16,32,64},
 * M * D <= 8192.  No reference code exists for this path: the algorithm is checked against autograd
 * through the dense definition (oracle/flare_oracle.py: causal_bwd_chunked, causal_bwd_autograd). */
size_t flare_causal_bwd_workspace_bytes(const FlareProblem* p);
int flare_causal_bwd(const FlareProblem* p, const void* q, const void* k, const void* v, const void* dy,
                     float* dq32, void* dk, void* dv, float* workspace, flare_stream_t stream);

/* Causal linear attention, Y_t = Q_t . sum_{n<=t} K_n^T V_n / N (lra/models/triton/causal_linear.py:23-145;
 * reference form :317-336; forward only, as there).  q, k: [B,H,N,Dk]; v, y: [B,H,N,Dv]; strides in
 * elements for dims (b, h, n), unit stride on the last dim.  workspace:
 * flare_causal_linear_workspace_bytes bytes.  Dk, Dv up to 256.  16-bit inputs with Dk = 128, Dv in {32, 64}
 * and 16-byte aligned rows run as three tensor-core passes over 128-token chunks; the rest on fp32 kernels. */
size_t flare_causal_linear_workspace_bytes(int B, int H, int N, int Dk, int Dv);
int flare_causal_linear(int B, int H, int N, int Dk, int Dv, int dtype, const void* q, const int64_t* q_stride,
                        const void* k, const int64_t* k_stride, const void* v, const int64_t* v_stride,
                        void* y, const int64_t* y_stride, float* workspace, flare_stream_t stream);

/* Triple attention (lra/models/triton/triple.py:27-290; einsum references :846-860, :887-931) as the two
 * shapes of work its forward and backward are made of.  Inputs are [BH, N, D] contiguous in `dtype`,
 * as the reference makes them (triple.py:51-55); tensors of rank 3 are fp32.
 *   flare_triple_outer:    out[bh][i][j][k] = alpha * sum_n a[n,i] b[n,j] c[n,k]   (STATE with alpha = 1/N,
 *                          dSTATE with alpha = 1).  Da in {16,32,64}; Db, Dc multiples of 4 up to 64.
 *                          workspace: flare_triple_workspace_bytes bytes.
 *   flare_triple_contract: out[bh][n][x] = alpha * sum_{y,z} T[x,y,z] a[n,y] b[n,z], where T[x,y,z] is read
 *                          at t + bh*Dx*Dy*Dz + x*sx + y*sy + z*sz (element strides: any permutation of a
 *                          contiguous [D0,D1,D2] tensor).  O, dQ1, dQ2, dK1, dK2, dV are all of this form.
 *                          Dz in {16,32,64}; Dx, Dy multiples of 4 up to 64. */
size_t flare_triple_workspace_bytes(int BH, int N, int Da, int Db, int Dc);
int flare_triple_outer(int BH, int N, int Da, int Db, int Dc, int dtype, const void* a, const void* b,
                       const void* c, float alpha, float* out, float* workspace, flare_stream_t stream);
int flare_triple_contract(int BH, int N, int Dx, int Dy, int Dz, int dtype, const float* t, int64_t sx,
                          int64_t sy, int64_t sz, const void* a, const void* b, float alpha, void* out,
                          flare_stream_t stream);

/* Reads (and optionally clears) the device status word of the current device; synchronises.
 * Non-zero means a kernel gave up on a bounded wait (bit 0: inside a tensor-core kernel; bit 1: a peer
 * did not arrive at flare_peer_barrier) and the output since the last clear is
 * not valid.  No counterpart in the reference.  `out` is a HOST pointer. */
int flare_device_status(int* out, int clear);

/* How many of the streaming passes (gather, scatter, dZ, main backward, per-token gradients, dQ) this
 * process has enqueued on the tensor-core kernels and on the fp32-arithmetic kernels since the library
 * was loaded; either pointer may be NULL.  Lets a caller (or a test) see which family served its
 * shapes.  HOST pointers.  No counterpart in the reference. */
int flare_pass_counts(long long* tensor_core, long long* simt);

/* Measurement aid, no counterpart in the reference: launches `blocks` x 256 threads that each
 * issue 8*iters dependent-chain ex2 operations, so that the benchmark can time the exponential
 * unit's peak on the device it runs on.  `out` is one device float (never written in practice). */
int flare_probe_ex2(int blocks, int iters, float* out, flare_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif  /* FLARE_B200_H_ */
