// Allocation-free entry point for the embedding backward update.
//
// This function has no counterpart in the reference: it exists for callers of this library that
// are not allowed to allocate device memory.  Examples are a serving process whose memory budget
// was fixed (and handed out) at start-up, code running between cudaMalloc-free phases of a host
// application that forbids allocator calls on its hot path, or an embedder that links this library
// without torch and therefore has no caching allocator to ask.  Every other entry point of the
// backward update takes a caller-provided scratch buffer that somebody had to allocate; this one
// brings its own.
//
//   int recml_emb_bwd_update_static(const BwdParams* p, long long max_occ, int gains,
//                                   cudaStream_t stream, char* err, int err_len);
//
// Same contract as recml_emb_bwd_update (sorted occurrence keys / values, gradient vectors, table
// and optimizer slots are passed in by the caller; `p->scratch` is ignored), with these differences:
//   * The kernel walks the sorted occurrences in ranges of RECML_EMB_STATIC_RANGE (128) entries.  The
//     scratch for runs of equal rows that cross range boundaries is a file-scope `static __device__`
//     array of RECML_EMB_STATIC_MAX_OCC/128 x RECML_EMB_STATIC_MAX_DIM floats (1 MiB).  It is part of
//     the library image: every GPU that loads the library holds it until the process exits.
//   * Limits: max_occ <= RECML_EMB_STATIC_MAX_OCC and p->dloc <= RECML_EMB_STATIC_MAX_DIM.  Larger
//     requests are refused with a negative return code and a message in `err` (when given).
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine.  The first call
//     on a device looks up the device address of the array (cudaGetSymbolAddress); make that first
//     call before starting any stream capture.
//   * All calls on a device share the one array.  The lines a call can touch are cleared at its
//     start (cudaMemsetAsync on `stream`), so calls issued in order on one stream are independent,
//     but two calls that overlap on the GPU (different streams, no ordering between them) race on the
//     array and give undefined results.
// Return value: 0 on success; -20 null parameters, -21 max_occ too large, -22 dim too large,
// -23 device query failed, -24 symbol lookup failed, -25 clearing failed, other negatives from the
// kernel launch.
#pragma once
#include <cuda_runtime.h>

#define RECML_EMB_STATIC_MAX_OCC 262144LL
#define RECML_EMB_STATIC_MAX_DIM 128
#define RECML_EMB_STATIC_RANGE 128

#ifdef __cplusplus
namespace recml { namespace emb { struct BwdParams; } }
extern "C" int recml_emb_bwd_update_static(const recml::emb::BwdParams* p, long long max_occ, int gains,
                                           cudaStream_t stream, char* err, int err_len);
#endif
