// An entry point of the tensor-core matrix product that allocates nothing.
//
// It has no counterpart in the reference (which has no CUDA code at all); it exists for
// users of this library who may not allocate device memory at the time they need a
// product: a host application that has handed the whole device to a pool of its own
// and forbids libraries to take more, a process that runs under a fixed memory budget
// and must know its footprint when it starts, or a latency-critical loop in which the
// device-wide synchronisation of cudaMalloc/cudaFree would stall every other stream.
//
// The ordinary entry point (gb_gemm_tc) gets the scratch memory in which CTAs that share an
// output tile leave their partial sums from the caller, who usually allocates it; this one
// uses a fixed array that lives in the library itself.  The caller still passes inputs and
// outputs.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch: floats of partial tiles, and tiles that CTAs may share.
// Every GPU that loads the library holds GB_NOALLOC_SCRATCH_FLOATS * 4 bytes (8 MiB) plus the
// counters until the process exits.
#define GB_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define GB_NOALLOC_COUNTERS 1024

// out[t,n] = sum_k X[t,k] * W[n,k] (+ bias[n]): X bf16 [T,K] with pitch ldx, W bf16 [N,K] with
// pitch ldw, out bf16 (dtype 1) or f32 (dtype 0) [T,N] with pitch ldo, bias f32 or bf16 or null.
// K and the pitches must be multiples of 8 and the pointers 16-byte aligned, as for gb_gemm_tc.
// Returns 0, or non-zero with a message in gb_last_error(): sizes whose partial tiles would need
// more than the built-in scratch are refused (gb_gemm_tc with caller memory takes them).
//
// It calls no cudaMalloc, cudaFree, or any other allocating routine, on the device or the host.
// The first call on each device looks up the address of the built-in scratch
// (cudaGetSymbolAddress, with that device current); make that first call before any stream
// capture begins on that device.  The kernel exists in five widths (tiles of 16, 32, 64, 128
// and 256 tokens, chosen from T and N), and the first launch of each width on each device
// loads that kernel and raises its shared-memory limit (cudaFuncSetAttribute): a caller who
// must not trigger even that later on, or who captures streams, warms up one call of every
// width it will use (T = 16, 32, 64 and so on) first.
// The launch is an ordinary one: it starts when everything before it on `stream` has finished,
// so W and X may be outputs of earlier work on the stream, of this entry point included.
// All calls share the one scratch array, and it keeps what the last call left: the counters
// that must start at zero are cleared on `stream` before each launch, the partial tiles are
// always written before they are read.  Two calls that overlap on the GPU (different streams,
// or different host threads) race on it; run them one after the other.
// Where CTAs share tiles of 32 tokens or more, each of them waits (for two seconds at most, then
// the status below is set) until the tile's other CTAs have stored their sums; the kernel never
// has more CTAs than the device holds at once, so they all run as soon as whatever occupied the
// SMs before has left.  Work on other streams that keeps SMs busy for seconds can make that wait
// run out.
int gb_gemm_tc_noalloc(const void* X, long long ldx, const void* W, long long ldw, const void* bias, int bias_dtype,
                       void* out, int out_dtype, long long ldo, int T, int N, int K, cudaStream_t stream);

// After synchronising the stream: non-zero if a bounded wait inside the kernel gave up during a
// gb_gemm_tc_noalloc call since the last query (the output is then invalid).  Clears the flag.
int gb_gemm_tc_noalloc_status(void);

#ifdef __cplusplus
}
#endif
