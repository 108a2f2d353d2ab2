// Internal launch entry points shared between the translation units of the library.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace rlxq {

int launch_dequant_f32(cudaStream_t stream, uint32_t scheme, const uint8_t* w, uint64_t n_elems, float* out);

int launch_matmul_generic(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w,
                          void* y, bool ybf, uint32_t m, uint32_t k, uint32_t n);

// Staged tensor-mode GEMV (m <= 8).
bool staged_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x, bool xbf);
size_t staged_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n);
int launch_gemv_staged(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w,
                       void* y, bool ybf, uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes);
// Integer (dp4a) GEMV (m <= 2).
bool int_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x);
size_t int_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n);
int launch_gemv_int(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w, void* y,
                    bool ybf, uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes);

// tcgen05 / tensor-memory GEMV (m <= 8): weights decoded to fp16 in tensor memory, activations as bf16 high / low rows.
int launch_split_hi_lo(cudaStream_t stream, const float* x, void* out, uint64_t rows, uint64_t k);
int launch_add_halves(cudaStream_t stream, const float* y2, void* y, bool ybf, uint64_t rows, uint64_t n);
int launch_swiglu_pair(cudaStream_t stream, const float* gu, void* h, uint32_t m, uint32_t f);
// A chain of dependent batch-1/2 GEMVs in one cooperative launch (gemv_int.cu, gemv_chain_kernel).
struct ChainLayer { const uint8_t* w; uint32_t k, n, swiglu; };
size_t chain_workspace_bytes(uint32_t scheme, const ChainLayer* layers, uint32_t nlayers, uint32_t m);
int launch_gemv_chain(cudaStream_t stream, uint32_t scheme, const ChainLayer* layers, uint32_t nlayers, const void* x, bool xbf,
                      void* y, bool ybf, uint32_t m, void* ws, size_t ws_bytes);
bool int_mma_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x);
// whether the format's down projection also exists as a kernel that pushes its tiles into peers' exchange buffers
bool int_push_supported(uint32_t scheme);
size_t int_mma_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n);
int launch_gemv_int_mma(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w, void* y,
                        bool ybf, uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes);
bool gemv_tc_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x, bool xbf);
size_t gemv_tc_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n);
int launch_gemv_tc(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w, void* y, bool ybf,
                   uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes);

// tcgen05 / tensor-memory GEMM (m > 8, bf16 activations).
bool gemm_tc_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x, bool xbf);
size_t gemm_tc_workspace_bytes(uint32_t m, uint32_t k, uint32_t n);
int launch_gemm_grouped(cudaStream_t stream, uint32_t scheme, const void* x, uint32_t x_rows, const uint8_t* w,
                        uint32_t num_slabs, float* y2, uint32_t k, uint32_t n, const void* groups, uint32_t group_tiles,
                        uint32_t tile_rows);
int launch_gemm_tc(cudaStream_t stream, uint32_t scheme, const void* x, const uint8_t* w, void* y, bool ybf,
                   uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes);

// One MoE decode row: the slab of the weight stack is chosen by *expert_sel on the device.
bool int_expert_supported(uint32_t scheme, uint32_t k, uint32_t n, const void* w, const void* x);
int launch_gemv_int_expert(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w_stack, void* y,
                           bool ybf, uint32_t k, uint32_t n, uint32_t num_experts, const float* expert_sel, void* ws,
                           size_t ws_bytes);

struct TpPush;   // tp_comm.cuh: the exchange buffers of a tensor-parallel group (null: plain output)
int launch_gemv_int_swiglu(cudaStream_t stream, uint32_t scheme, const float* gu, const uint8_t* w, void* y, bool ybf,
                           uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes, const TpPush* tp = nullptr);

int staged_device_error(int* value);   // synchronises the device
int* static_error_word_if_resolved();  // error word inside the library image, once an allocation-free call resolved it
int staged_prepare_device();           // allocates the per-device error word (call outside capture)

// Shape-based selection used by rlxq_matmul / rlxq_workspace_bytes.
size_t matmul_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, uint32_t x_dtype, uint32_t y_dtype);
int dispatch_matmul(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w, void* y,
                    bool ybf, uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes);

}  // namespace rlxq
