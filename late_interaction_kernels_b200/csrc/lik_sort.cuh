// Stable sort of (key, value) pairs of 32-bit words on the device, and the offsets of the runs of equal keys.
// Used to group a pair list by query and by document for the deterministic backward.
#pragma once

#include "lik_common.cuh"

namespace lik {

// bytes of scratch stable_sort_pairs needs for n pairs (two alternate arrays and the digit histograms)
size_t sort_pairs_scratch(long long n);

// Sorts (keys, vals) by key, ascending, stable, 8 bits per pass over the low `key_bits` bits.  The sorted pairs
// end up in (keys, vals) themselves.  scratch: sort_pairs_scratch(n) bytes.
int stable_sort_pairs(unsigned* keys, unsigned* vals, long long n, int key_bits, void* scratch, cudaStream_t st);

// start[i] = number of sorted keys < i, for i in [0, n_seg]: the run of key i is [start[i], start[i + 1]).
int run_starts(const unsigned* sorted_keys, long long n, int n_seg, int* start, cudaStream_t st);

}  // namespace lik
