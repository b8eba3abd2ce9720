// host.h -- host-side helpers shared by the translation units of the library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ill {

// Records E as the calling thread's last CUDA error and returns ILL_ERR_CUDA.
int cuda_fail(cudaError_t e);

// Address of the current device's status word (a __device__ variable of the
// library; no allocation).  Null if the address cannot be taken.
unsigned int* device_status_word();

// Whether launches carry the programmatic-stream-serialization attribute.
bool pdl_enabled();

// Launch FN (grid, block, dynamic shared bytes) on ST with ARGS, with the
// programmatic-dependent-launch attribute when enabled.
int launch_kernel(const void* fn, dim3 grid, dim3 block, size_t smem, void** args, cudaStream_t st);

enum { MODE_PLAIN = 0, MODE_GLU = 1, MODE_MOE_GLU = 2,
       MODE_PEERS = 3 /* a plain one-token product whose results go to every rank's buffer, then the ranks meet */ };

// The matvec family's common entry (mv.cu): NMAT matrices of one format sharing
// the activations; NSEG segments when PTRS (a device table of base addresses)
// is given.  See ill_mv / ill_moe_mv for the argument meaning.
int mv_common(int fmt, int mode, int nmat, const uint64_t* w, const int* rows, int cols, uint64_t xq, uint64_t xs,
              uint64_t xsum, const uint64_t* y, const uint64_t* bias, int acc, int n, uint64_t ptrs, int nseg,
              long long add, long long up_add, int x_seg, long long y_seg, uint64_t seg_w, float clamp, void* stream);

// Lanes a row and units a lane of the one-token product for rows of UNITS units (mv.cu); false when a row does
// not fit in registers.  BIG: the launch moves 16 MB or more.
bool mv_pick_lanes(int fmt, int units, bool glu, bool big, int* lanes, int* upt);

// The several-token product on the tensor cores (mvt.cu); ILL_ERR_UNSUPPORTED where it has no kernel.
int mvt_try(int fmt, uint64_t w, int rows, int cols, uint64_t xq, uint64_t xs, uint64_t xsum, uint64_t y, uint64_t bias, int acc,
            int n, void* stream);
// the same for a chunk of tokens (more than 16): mmd.cu
int mmd_try(int fmt, uint64_t w, int rows, int cols, uint64_t xq, uint64_t xs, uint64_t xsum, uint64_t y, uint64_t bias, int acc,
            int n, void* stream);
// up to 16 tokens of rows with many columns, the columns dealt to a CTA's warps: mmd.cu
int mmk_try(int fmt, uint64_t w, int rows, int cols, uint64_t xq, uint64_t xs, uint64_t xsum, uint64_t y, uint64_t bias, int acc,
            int n, void* stream);

}  // namespace ill
