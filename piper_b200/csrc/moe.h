// Host-side launchers of the mixture-of-experts kernels (moe.cu): router,
// token permutation into padded expert segments, weighted combine, and their
// backward passes.  Conventions: T tokens, E experts, k experts per token;
// entry (t, j) is the j-th choice of token t; pos[t*k + j] is the row that
// entry occupies in the expert-sorted row buffer.
#pragma once
#include <cuda_runtime.h>

namespace piper {

// softmax over E logits per token, top-k, optional renormalisation of the k
// weights; counts[e] (int32, must be zero on entry) receives the number of
// entries routed to expert e.  E <= 256, k <= 8.
int moe_route(const void* logits_bf16, float* weights, int* idx, int* counts, long long T, int E, int k,
              int renorm, cudaStream_t st);

// d logits from d weights (fp32 [T, k]); recomputes the softmax.
int moe_route_bwd(const void* logits_bf16, const int* idx, const float* weights, const float* dweights,
                  void* dlogits_bf16, long long T, int E, int k, int renorm, cudaStream_t st);

// Group table for a [sources, experts] count matrix laid out source-major:
// g_len[g] = counts[g] rounded up to 128, g_start = exclusive prefix sum of
// g_len starting at row_base[source] when row_base != nullptr (region layout)
// or running over all groups otherwise.  total[0] = one past the last row.
int moe_group_table(const int* counts, int num_groups, int experts, const int* row_base, int* g_start,
                    int* g_len, int* total, cudaStream_t st);

// Every kernel below that indexes a row buffer through pos or a group table checks the index against rows_cap
// (rows of that buffer): a bad index is skipped and recorded in the status word.
//
// rows[pos] = x[t] for every entry; cursor (int32 [E], zero on entry) hands
// out positions inside each expert's segment; padding rows of every segment
// are zeroed.  Writes pos[T*k].
int moe_permute(const void* x_bf16, const int* idx, const int* g_start, const int* g_len, const int* counts,
                int* cursor, int* pos, void* rows_bf16, long long T, int D, int E, int k, long long rows_cap,
                int* status, cudaStream_t st);

// dx[t] = sum_j drows[pos[t*k+j]]
int moe_permute_bwd(const void* drows_bf16, const int* pos, void* dx_bf16, long long T, int D, int k,
                    long long rows_cap, int* status, cudaStream_t st);

// out[t] = sum_j weights[t, j] * rows[pos[t*k+j]]
int moe_combine(const void* rows_bf16, const int* pos, const float* weights, void* out_bf16, long long T, int D,
                int k, long long rows_cap, int* status, cudaStream_t st);

// drows[pos] = weights[t, j] * dout[t]; dweights[t, j] = <rows[pos], dout[t]>; padding rows of drows
// (described by the group table) are zeroed.
int moe_combine_bwd(const void* rows_bf16, const void* dout_bf16, const int* pos, const float* weights,
                    void* drows_bf16, float* dweights, const int* g_start, const int* g_len, const int* counts,
                    int num_groups, long long T, int D, int k, long long rows_cap, int* status, cudaStream_t st);

}  // namespace piper
