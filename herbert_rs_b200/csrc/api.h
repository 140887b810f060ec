// C interface of libherbert_b200: one launcher per kernel.  All pointers are device pointers
// unless a name ends in _host; `stream` is a cudaStream_t.  Return value 0 = launched,
// otherwise hb_last_error() holds the reason and nothing was launched.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

const char* hb_last_error(void);
int hb_abi_version(void);

// dtype codes used where one entry point serves both paths
#define HB_F32 0
#define HB_BF16 1

// epilogues of the matrix products
#define HB_EPI_STORE 0      // C (activation dtype) = A W^T
#define HB_EPI_STORE_F32 1  // C (float)            = A W^T
#define HB_EPI_RESIDUAL 2   // C (float)           += A W^T

#ifdef __cplusplus
}
#endif
