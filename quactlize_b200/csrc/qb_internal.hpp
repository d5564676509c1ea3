// Internal launch interfaces between the translation units of libquactlize_b200 (not part of the C ABI).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace qb {

int enqueue_native_gemv(uint8_t const* blocks, __half const* x, float* out, int const* offsets,
                        int n, int bpr, int experts, int m_rows, int max_rows, int qtype, bool per_row_x,
                        bool force_generic, cudaStream_t stream);
bool enqueue_q4k_gemv1(uint8_t const* blocks, __half const* x, float* out, int const* offsets, int n, int bpr,
                       int experts, int rows, int max_rows, unsigned int* status, cudaStream_t stream);
bool enqueue_q4k_gemv1_dual(uint8_t const* blocks1, int n1, uint8_t const* blocks2, int n2, __half const* x, float* out1, float* out2,
                            int bpr, unsigned int* status, cudaStream_t stream);   // two matrices, one activation row, one launch
bool enqueue_q4k_mma(uint8_t const* blocks, __half const* x, float* out, int const* offsets, int n, int bpr, int experts,
                     int rows, unsigned int* status, cudaStream_t stream);   // tensor-core small-batch form
bool enqueue_q4k_rows(uint8_t const* blocks, __half const* x, float* out, int n, int bpr, int rows, unsigned int* status,
                      cudaStream_t stream);                 // dense, 1..8 rows, tensor cores on the single-row kernel's copy structure
bool enqueue_kquant_gemv1(uint8_t const* blocks, __half const* x, float* out, int const* offsets, int n, int bpr, int experts,
                          int rows, int max_rows, int qtype, unsigned int* status, cudaStream_t stream);   // Q2_K/Q3_K/Q5_K/Q6_K, one row per pass
bool enqueue_dequantize(uint8_t const* blocks, __half* out, int count, int qtype, cudaStream_t s);
bool enqueue_unpack(uint8_t const* blocks, int8_t* codes, __half* scale, __half* zero, int count, int qtype, cudaStream_t s);
// planes (Native order) + fp16 scale/zero planes -> fp16 [E][n][k]; `shift` is added to the unsigned code
bool enqueue_planes_dequantize(uint8_t const* low, uint8_t const* high, __half const* scale, __half const* zero, __half* out,
                               int experts, int n, int k, int lo, int hi, int gs, int shift, cudaStream_t s);
bool enqueue_prepass(uint8_t const* sblocks, uint16_t const* d, uint16_t const* dmin, int count, int qtype, int zmul,
                     __half* scale, __half* zero, cudaStream_t s);
bool enqueue_prepass_unit(uint8_t const* units, __half* scale, __half* zero, int experts, int n, int nsb, int qtype,
                          int zmul, cudaStream_t s);

// Plane GEMV.  scale_mode: 0 = fp16 planes scale(+zero) [E][K/gs][N]; 1 = packed k-quant units of `qtype`.
struct PlaneGemvDesc {
  void const* act;            // fp16 or bf16 [rows][k]
  uint8_t const* low;         // [E][n][k*lo_bits/8]
  uint8_t const* high;        // [E][n][k*hi_bits/8] or nullptr
  void const* scale;          // fp16 [E][k/gs][n]    (scale_mode 0)
  void const* zero;           // fp16 [E][k/gs][n] or nullptr
  uint8_t const* units;       // [E][k/256/P][n][unit_total] (scale_mode 1)
  void* out;                  // fp16 / bf16 / fp32 [rows][n]
  int const* offsets;         // cumulative [experts+1] or nullptr
  int n, k, experts, m_rows, max_rows;
  int lo_bits, hi_bits, group_size, scale_mode, qtype;
  int code_offset;            // added to the unsigned code before scaling (e.g. -8), 0 if none
  int act_bf16;               // activations are bf16 (else fp16)
  int out_kind;               // 0 = fp16, 1 = fp32, 2 = bf16
};
int enqueue_plane_gemv(PlaneGemvDesc const& d, cudaStream_t stream);   // 0 ok, 40 unsupported shape
int enqueue_rowthread_gemv(PlaneGemvDesc const& d, cudaStream_t stream);   // row-thread form; 40 = shape not covered by it
int enqueue_rowmma_gemv(PlaneGemvDesc const& d, cudaStream_t stream);      // tensor-core small-batch form; 40 = not covered
int enqueue_bc_gemv1(PlaneGemvDesc const& d, cudaStream_t stream);         // planes + packed units, one activation row per weight pass; 40 = not covered

// Tensor-core mixed-input GEMM (dense when experts == 0, else grouped with cumulative offsets).
struct GemmDesc {
  void const* act;            // fp16 or bf16 [total_rows][k]
  uint8_t const* low;         // [E][n][k*lo_bits/8]
  uint8_t const* high;        // [E][n][k*hi_bits/8] or nullptr
  void const* scale;          // fp16 [E][k/gs][n]
  void const* zero;           // fp16 [E][k/gs][n] or nullptr
  void* out;                  // act dtype [total_rows][n]
  int const* offsets;         // cumulative device int [experts+1] (grouped)
  int total_rows, n, k, experts, group_size, lo_bits, hi_bits, code_offset, act_bf16;
  int tile;                   // 0 = chosen from the problem size, 128 / 256 = that CTA tile (the two compiled tactics)
  int splits;                 // split-K slices; 0 or 1 = none.  > 1 needs `partial` and at most k/128 slices
  float* partial;             // fp32 [splits][total_rows][n] workspace of the split-K form (caller-owned)
  int shallow;                // 1 = the decode tactic: 128 x 128 tiles with two-deep rings (several CTAs per SM)
  unsigned long long const* out_rows;   // optional device array [total_rows]: where each output row goes (see GemmArgs)
};
// Split-K slices that fill the SMs for a decode-sized grouped problem: row_tiles is the number of (expert, row tile)
// pairs that hold rows (an upper bound is fine).  1 when the plain launch already gives every SM a tile.
int splitk_auto(int row_tiles, int n, int k);
int enqueue_mixed_gemm(GemmDesc const& d, cudaStream_t stream);    // 0 ok, 30/33 refused, 41 runtime
long long gemm_swap_launches();                                    // launches of the swapped (TMEM-operand) form so far

}  // namespace qb
