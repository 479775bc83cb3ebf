// Declarations shared by the translation units of libunholy_pkv.so that are NOT part of its C ABI (C++ linkage, hidden
// visibility): the calling thread's error message, the top-k path knob, and the one-launch top-k's host entry points.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <string>

extern thread_local std::string pkv_g_err;  // what pkv_last_error() returns (defined in pkv_kernels.cu)
extern int pkv_g_topk_path;                 // pkv_tune knob 7 (defined in pkv_kernels.cu)

// pkv_topk_cluster.cu: the whole top-k selection in one launch of thread-block clusters, for the shapes it takes.
struct pkv_topk_cluster_group {
  long long off, ld, idx_off;
  int rows, n, k, row0;
};
bool pkv_topk_cluster_eligible(int T, int n, int k);
int pkv_topk_cluster_launch(const uint16_t* scores, const pkv_topk_cluster_group* groups, int ngroups, int32_t* idx,
                            cudaStream_t stream, bool* usable, std::string& err);
