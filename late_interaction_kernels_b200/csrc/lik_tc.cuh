// Interface between the C-ABI entry points and the tcgen05 scoring kernel (lik_fwd_tc.cu).
#pragma once

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

}  // namespace lik
