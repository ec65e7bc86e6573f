// Internal launch functions shared by the C-ABI layer and the kernel files.
#pragma once
#include "common.cuh"

namespace flare {

// fp32-arithmetic SIMT family (flare_simt.cu)
int simt_gather_partial(const Ctx& c, int dtype, const void* q, const void* k, const void* v,
                        const uint8_t* mask, float* rec, cudaStream_t st);
int simt_dz_partial(const Ctx& c, int dtype, const void* q, const void* k, const void* dy,
                    const uint8_t* mask, const float* lse_n, float* dz_part, cudaStream_t st);
int simt_dq_partial(const Ctx& c, int dtype, const void* q, const void* k, const void* v, const void* dy,
                    const uint8_t* mask, const float* z32, const float* dz32, const float* lse_m,
                    const float* lse_n, const float* delta_n, float* dq_part, cudaStream_t st);
int simt_scatter(const Ctx& c, int dtype, const void* q, const void* k, const float* z32,
                 const uint8_t* mask, void* y, float* lse_n, cudaStream_t st);
int simt_bwd_tokens(const Ctx& c, int dtype, const void* q, const void* k, const void* v, const void* dy,
                    const void* y, const uint8_t* mask, const float* z32, const float* dz32,
                    const float* lse_m, const float* lse_n, void* dk, void* dv, float* delta_n,
                    cudaStream_t st);
int launch_combine(const float* rec, int n_parts, long long rows, int D, int dtype, float* z32,
                   void* z_out, float* lse_m, float* rec_out, cudaStream_t st);
int launch_reduce_sum(const float* parts, int n_parts, long long n, float* out, cudaStream_t st);
int launch_combine_ptrs(const float* const* recs, int n_parts, long long rows, int D, int dtype, float* z32,
                        void* z_out, float* lse_m, float* rec_out, cudaStream_t st);
int launch_reduce_sum_ptrs(const float* const* parts, int n_parts, long long n, float* out, cudaStream_t st);
int launch_probe_ex2(int blocks, int iters, float* out, cudaStream_t st);
int launch_peer_barrier(int32_t* const* flags, int rank, int world, int epoch, cudaStream_t st);


// tcgen05 tensor-core family (flare_tc_*.cu): bf16, D in {16,32,64}, M a multiple of 32 up to 256.
// Each launcher returns FLARE_EUNSUPPORTED when the driver rejects a tensor map; the caller
// then uses the SIMT kernel for that pass.
bool tc_scatter_supported(const Ctx& c, int dtype);
int tc_scatter(const Ctx& c, const void* q, const void* k, const float* z32, const uint8_t* mask, void* y,
               float* lse_n, cudaStream_t st);
// decoupled-schedule scatter (one CTA per SM, two tiles in flight; D <= 32)
bool tc_scatter2_supported(const Ctx& c, int dtype);
int tc_scatter2(const Ctx& c, int dtype, const void* q, const void* k, const float* z32, const uint8_t* mask, void* y,
                float* lse_n, cudaStream_t st);
bool tc_lat_supported(const Ctx& c, int dtype);
int tc_gather_partial(const Ctx& c, const void* q, const void* k, const void* v, float* rec, cudaStream_t st);
int tc_dz_partial(const Ctx& c, const void* q, const void* k, const void* dy, const float* lse_n, float* dz_part,
                  cudaStream_t st);
// decoupled-schedule versions of the two latent-major passes (D <= 32)
bool tc_lat2_supported(const Ctx& c, int dtype);
int tc_gather_partial2(const Ctx& c, int dtype, const void* q, const void* k, const void* v, const uint8_t* mask,
                       float* rec, cudaStream_t st);
int tc_dz_partial2(const Ctx& c, int dtype, const void* q, const void* k, const void* dy, const uint8_t* mask,
                   const float* lse_n, float* dz_part, cudaStream_t st);
bool tc_bwd_supported(const Ctx& c, int dtype);
// the general tensor-core backward: bf16/fp16, mask, either softmax term, latents in blocks of 256;
// flag (or null): run only the (b, h) whose flag is 1
int tc_bwd_main(const Ctx& c, int dtype, const void* q, const void* k, const void* v, const void* dy, const void* y,
                const uint8_t* mask, const float* z32, const float* dz32, const float* lse_m, const float* lse_n,
                void* dk, void* dv, float* dq_part, const int* flag, cudaStream_t st);
// The one-exponential form of the plain case (bf16, both terms, no mask, D = 32) behind an on-device range
// check that selects, per (b, h), between it (flag 0) and the general kernel above (flag 1).
size_t tc_bwd_fast_scratch_bytes(const Ctx& c);
int tc_bwd_fast_main(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                     const float* z32, const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                     float* dq_part, void* scratch, const int** flag_out, cudaStream_t st);
// the one-exponential kernel itself: 128-latent steps, S^T double-buffered, T' single, two issuing warps
bool tc_bwd_fast_supported(const Ctx& c, int dtype);
int tc_bwd_fast_launch(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                   const float* z32, const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                   float* dq_part, const float* mu, const int* flag, cudaStream_t st);
// per-device host state (tc_runtime.cu)
int tc_read_status(int* out, bool clear);
int* tc_status_ptr();
int num_sms();
int tc_set_dyn_smem(const void* kernel, int bytes);

// Causal prefill, pass 3 on the tensor cores (flare_causal_tc.cu): bf16, M <= 128, D in {32, 64}.
bool causal_tc_walk_supported(const FlareProblem* p, const void* q, const void* k, const void* v, const void* y);
// pass 1 for the same shapes: the record of every 128-token chunk on its own, racc [chunks][B][H][M][D] in 16 bits and
// rml [chunks][B][H][M] = (m, l); the scan turns them into the prefixes in place
int causal_tc_record(const FlareProblem* p, const void* q, const void* k, const void* v, __nv_bfloat16* racc, float2* rml,
                     int chunks, cudaStream_t st);
// redo: int [chunks][B*H], written by every CTA: 1 where the chunk must be redone by the fp32 walk.
// pacc [chunks][B][H][M][D] bf16 and pml [chunks][B][H][M] (m, l): the prefix of every chunk as the scan wrote it.
int causal_tc_walk(const FlareProblem* p, const void* q, const void* k, const void* v, void* y, const __nv_bfloat16* pacc,
                   const float2* pml, int* redo, int chunks, cudaStream_t st);

// Causal linear attention on the tensor cores (flare_causal_linear_tc.cu): 16-bit inputs, Dk = 128, Dv in {32, 64}.
bool causal_linear_tc_supported(int B, int H, int N, int Dk, int Dv, int dtype, const void* q, const int64_t* qs,
                                const void* k, const int64_t* ks, const void* v, const int64_t* vs, const void* y,
                                const int64_t* ys);
size_t causal_linear_tc_workspace(int B, int H, int N, int Dk, int Dv);
int causal_linear_tc(int B, int H, int N, int Dv, int dtype, const void* q, const int64_t* qs, const void* k,
                     const int64_t* ks, const void* v, const int64_t* vs, void* y, const int64_t* ys, float* workspace,
                     cudaStream_t st);

// Triple attention on the tensor cores (flare_triple_tc.cu): 16-bit inputs, every feature dimension 32.
bool triple_tc_supported(int N, int D0, int D1, int D2, int dtype);
bool triple_tc_strides_ok(long long sx, long long sy, long long sz);
size_t triple_tc_outer_workspace(int BH, int N);
int triple_tc_outer(int BH, int N, int dtype, const void* a, const void* b, const void* c, float alpha, float* out,
                    float* ws, cudaStream_t st);
int triple_tc_contract(int BH, int N, int dtype, const float* t, long long sx, long long sy, long long sz, const void* a,
                       const void* b, float alpha, void* out, cudaStream_t st);

}  // namespace flare
