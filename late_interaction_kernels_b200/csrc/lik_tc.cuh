// Interface between the C-ABI entry points and the tcgen05 scoring kernel (lik_fwd_tc.cu).
#pragma once

#include <cuda.h>

#include "lik_common.cuh"
#include "lik_plaid_row.cuh"

namespace lik {

// What a launch does beyond lik_fwd_args: fused top-k instead of a score matrix, documents decoded from a
// compressed index instead of loaded.
struct TcExtra {
  int topk_k = 0;  // > 0: keep the k best documents per query, merged into topk_scores / topk_index [n_q, k]
  int topk_largest = 1;
  long long topk_index_offset = 0;
  float* topk_scores = nullptr;
  int64_t* topk_index = nullptr;
  int topk_flags = 0;     // LIK_TOPK_CONTINUE / LIK_TOPK_PARTIAL
  int topk_doc_base = 0;  // index of this call's first document in the corpus
  const PlaidSrc* plaid = nullptr;
};

bool fwd_tc_supported(const lik_fwd_args& a);
bool fwd_tc_topk_supported(const lik_fwd_args& a, const TcExtra& x);
bool fwd_tc_plaid_supported(const lik_fwd_args& a, const TcExtra& x);
size_t fwd_tc_workspace(const lik_fwd_args& a, const TcExtra& x);
int launch_fwd_tc(const lik_fwd_args& a, const float* qn, const float* dn, void* ws, size_t ws_bytes, cudaStream_t st,
                  const TcExtra& x);


// Shared with the document-head kernel (lik_head.cu).
constexpr int LEN_FLAG_MASKED = 1 << 30;  // effective length of a document whose mask is not a plain prefix
int make_tmap_rows(CUtensorMap* map, const void* data, int dtype, long long inner, long long n_rows, long long row_stride,
                   int box_rows);
bool tmap_available();
// out[j] = (1 + index of the last valid token of padded document j) | LEN_FLAG_MASKED when the valid tokens are not a prefix
int launch_mask_lens(const unsigned char* mask, const int* lens, int n_seq, int max_len, long long seq_stride, int* out,
                     cudaStream_t st);

}  // namespace lik
