/* C ABI of libquactlize_b200.so -- the B200 (sm_100a) device library behind quactlize's raw-pointer boundary.
 *
 * The library is a drop-in for the reference's device library: every `quactlize_ppu_*` entry below has the name,
 * argument list, argument meaning and return-code behaviour of the reference symbol it replaces (cited per entry as
 * file:line inside the reference project), so the reference's own host extension can dlopen this file through
 * QUACTLIZE_PPU_LIB (quactlize/csrc/preprocess/thop/ppu_backend.cpp:58-134 resolves exactly these names).
 * `quactlize_b200_*` entries are additive: they cover what the reference reaches only through C++ templates
 * (generic per-group W4/W2/W1 planes, bf16 activations, multi-row raw-block GEMV, device-pointer MoE forms).
 *
 * Conventions (quactlize/csrc/preprocess/thop/ppu_backend.h:23-104, quactlize/include/quactlize_ppu_device.h:12-51):
 *   - raw pointers and ints only; fp16/bf16 cross as uint16_t*; qtype is the ggml number (Q2_K=10 .. Q6_K=14);
 *   - host-pointer entries take HOST memory: they allocate device temporaries, copy in, launch, synchronise, copy out;
 *   - `_dev_` entries take DEVICE memory and a native stream cast to void* (NULL = default stream); a zero return
 *     means ENQUEUED, not completed; they neither allocate nor synchronise; the caller owns every buffer;
 *   - every entry returns an int: 0 ok, small distinct codes for refused arguments, 41 for a latched runtime failure
 *     (allocation / copy / launch / synchronise / bounded device wait), never an exception or abort; host outputs are
 *     untouched on failure;
 *   - weights: raw GGUF k-quant blocks [E][N][K/256][block bytes] row-major by output row, or the offline artifact:
 *     Native code planes low [E][N][K*lo/8], high [E][N][K*hi/8] (element k of a row at bit k*bits, LSB first;
 *     Q3_K/Q6_K offset-binary) plus either fp16 planes scale/zero [E][K/gs][N] or packed units
 *     [E][K/256/P][N][P*sb_bytes];  grouped activations/outputs are concatenated in expert order with cumulative
 *     int offsets[E+1].
 */
#ifndef QUACTLIZE_B200_H_
#define QUACTLIZE_B200_H_

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- config inventory records: quactlize/include/quactlize_ppu_config.h:12-40 ----------------------------------- */
typedef struct quactlize_ppu_config_v1 {
  bool enable_cuda_kernel;
  char const* name;
  int32_t tile_m, tile_n, warp_m, warp_n, stages;
} quactlize_ppu_config_v1;

typedef struct quactlize_ppu_config_v2 {
  bool enable_cuda_kernel;
  char const* name;
  int32_t tile_m, tile_n, tile_k, warp_m, warp_n, stages;
} quactlize_ppu_config_v2;

/* ================================ raw GGUF block consumers (CUDA-core family) =================================== */

/* Independent block rows, each with its own activation slice: blocks [rows*bpr][block_bytes], x fp16
 * [rows*bpr*256], out fp32 [rows].  Replaces quactlize/csrc/device/ppu_backend.cu:297-304. */
int quactlize_ppu_vecdot(uint8_t const* blocks, int64_t block_bytes, uint16_t const* x, float* out,
                         int rows, int blocks_per_row, int qtype);
/* Dense decode GEMV, one shared activation x fp16 [bpr*256], out fp32 [rows].  ppu_backend.cu:306-313. */
int quactlize_ppu_vecdot_dense(uint8_t const* blocks, int64_t block_bytes, uint16_t const* x, float* out,
                               int rows, int blocks_per_row, int qtype);
/* Device-pointer form.  ppu_backend.cu:315-326, quactlize/include/quactlize_ppu_device.h:15-17. */
int quactlize_ppu_vecdot_dense_dev_v1(uint8_t const* blocks, int64_t block_bytes, uint16_t const* x, float* out,
                                      int rows, int blocks_per_row, int qtype, void* stream);
/* Ragged MoE decode: blocks [E][n][bpr][bytes], gathered x [total_rows][bpr*256], offsets [E+1], out fp32
 * [total_rows][n].  ppu_backend.cu:373-396. */
int quactlize_ppu_vecdot_moe(uint8_t const* blocks, int64_t block_bytes, uint16_t const* x, int const* row_offsets,
                             float* out, int n, int blocks_per_row, int experts, int total_rows, int max_rows, int qtype);
int quactlize_ppu_vecdot_moe_config_v1(uint8_t const* blocks, int64_t block_bytes, uint16_t const* x, int const* offsets,
                                       float* out, int n, int blocks_per_row, int experts, int total_rows, int max_rows,
                                       int qtype, char const* config_name);
/* ppu_backend.cu:348-371 */
int32_t quactlize_ppu_vecdot_moe_config_valid_v1(int total_rows, int n, int k, int group_size, int experts, int max_rows,
                                                 int qtype, char const* config_name);
int32_t quactlize_ppu_list_valid_vecdot_moe_configs_v2(quactlize_ppu_config_v2* configs, int32_t capacity, int total_rows,
                                                       int n, int k, int group_size, int experts, int max_rows, int qtype);
/* Raw blocks [n_blocks][bytes] -> fp16 [n_blocks][256], bit-exact half(dl*q - ml).  ppu_backend.cu:433-439. */
int quactlize_ppu_dequantize(uint8_t const* blocks, int64_t block_bytes, uint16_t* out, int n_blocks, int qtype);
/* Scale blocks + fp16 headers -> fp16 (scale, zero) [n][groups]; zmul in {0, 8}.  ppu_backend.cu:441-452. */
int quactlize_ppu_prepass(uint8_t const* blocks, int64_t block_bytes, uint16_t const* d, uint16_t const* dmin, int n,
                          uint16_t* scale, uint16_t* zero, int groups, int qtype, int zmul);
/* Packed units [E][unit][N][bytes] -> fp16 planes [E][K/gs][N]; zmul in {-32,-24,-4,0,8}.  ppu_backend.cu:454-467. */
int quactlize_ppu_prepass_unit(uint8_t const* units, uint16_t* scale, uint16_t* zero, int n, int k, int experts,
                               int qtype, int zmul);

/* additive: m >= 1 shared activation rows x fp16 [m][k], out fp32 [m][rows]; force_generic selects the simple
 * warp-per-row kernel.  No counterpart entry in the reference (its dense entry is m = 1, ppu_backend.cu:93-106). */
int quactlize_b200_vecdot_rows_dev_v1(uint8_t const* blocks, int64_t block_bytes, uint16_t const* x, float* out, int m,
                                      int rows, int blocks_per_row, int qtype, int force_generic, void* stream);
/* additive device-pointer forms of the entries above */
/* Two raw-block matrices [n_a][bpr] and [n_b][bpr] of one format against ONE fp16 activation row in one launch (a layer's
 * gate and up projections): out_a fp32 [n_a], out_b fp32 [n_b].  Device pointers, enqueue only; codes as vecdot_dense. */
int quactlize_b200_vecdot_dense2_dev_v1(uint8_t const* blocks_a, int n_a, uint8_t const* blocks_b, int n_b, int64_t block_bytes,
                                        uint16_t const* x, float* out_a, float* out_b, int bpr, int qtype, void* stream);
int quactlize_b200_vecdot_dev_v1(uint8_t const* blocks, int64_t block_bytes, uint16_t const* x, float* out, int rows,
                                 int blocks_per_row, int qtype, void* stream);
int quactlize_b200_vecdot_moe_dev_v1(uint8_t const* blocks, int64_t block_bytes, uint16_t const* x, int const* offsets,
                                     float* out, int n, int blocks_per_row, int experts, int total_rows, int max_rows,
                                     int qtype, void* stream);
int quactlize_b200_dequantize_dev_v1(uint8_t const* blocks, int64_t block_bytes, uint16_t* out, int n_blocks, int qtype,
                                     void* stream);
int quactlize_b200_prepass_unit_dev_v1(uint8_t const* units, uint16_t* scale, uint16_t* zero, int n, int k, int experts,
                                       int qtype, int zmul, void* stream);

/* ================================ bit-plane GEMV (scale-first and merged artifact) ============================== */

/* Scale-first GEMV over (low, high, scale, zero): out fp16 [total_rows][n]; experts == 0 is dense, otherwise offsets
 * is [E+1].  W = u*scale + zero with u the offset-binary plane code.  ppu_backend.cu:462-474. */
int quactlize_ppu_gemv_lowbit(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                              uint16_t const* zero, uint16_t* out, int total_rows, int n, int k, int group_size,
                              int qtype, int experts, int const* row_offsets, int max_rows);
/* ppu_backend.cu:476-489 */
int quactlize_ppu_gemv_lowbit_config_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                        uint16_t const* scale, uint16_t const* zero, uint16_t* out, int m, int n, int k,
                                        int group_size, int qtype, char const* config_name);
/* ppu_backend.cu:328-346 */
int32_t quactlize_ppu_gemv_lowbit_config_valid_v1(int m, int n, int k, int group_size, int qtype, char const* config_name);
/* ppu_backend.cu:491-509, quactlize_ppu_device.h:21-24 */
int quactlize_ppu_gemv_lowbit_dev_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                     uint16_t const* zero, uint16_t* out, int m, int n, int k, int group_size, int qtype,
                                     void* stream, char const* config_name);
/* Merged artifact (planes + packed units) GEMV, out fp32; experts == 0 requires total_rows == 1.
 * ppu_backend.cu:398-431, quactlize_ppu_device.h:28-32. */
int quactlize_ppu_bc_gemv(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint8_t const* units,
                          int const* row_offsets, float* out, int total_rows, int n, int k, int experts, int max_rows,
                          int qtype);
int quactlize_ppu_bc_gemv_dev_v1(uint16_t const* x, uint8_t const* low, uint8_t const* high, uint8_t const* units,
                                 int const* offsets, float* out, int total_rows, int n, int k, int experts, int max_rows,
                                 int qtype, void* stream);

/* additive: ragged MoE scale-first GEMV on device pointers (the reference reaches it only through its host entry). */
int quactlize_b200_gemv_lowbit_moe_dev_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                          uint16_t const* scale, uint16_t const* zero, uint16_t* out, int total_rows,
                                          int n, int k, int group_size, int qtype, int experts, int const* offsets,
                                          int max_rows, void* stream);
/* additive: generic per-group plane GEMV.  W = (lo + 2^bits_lo*hi + code_offset)*scale + zero (zero may be NULL);
 * bits_lo in {1,2,4}, bits_hi in {0,1,2}; act_dtype 0 = fp16, 1 = bf16; out_dtype 0 = fp16, 1 = fp32, 2 = bf16;
 * experts == 0 is dense over total_rows activation rows.  The reference instantiates these shapes only as C++
 * templates (tests/test_gemv_lowbit.cu:454-461, quactlize/include/gemv_lowbit/gemv_launcher.hpp:116-208). */
int quactlize_b200_gemv_plane_dev_v1(void const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                     uint16_t const* zero, void* out, int total_rows, int n, int k, int bits_lo,
                                     int bits_hi, int group_size, int code_offset, int act_dtype, int out_dtype,
                                     int experts, int const* offsets, int max_rows, void* stream);

/* ================================ tensor-core mixed-input GEMM (dense fpA_intB, MoE grouped) ===================== */

/* Config inventory.  quactlize/include/quactlize_ppu_config.h:42-71, quactlize/csrc/device/ppu_dense_backend.cu:603-664.
 * Two tensor-core tactics are listed ("256x256x64:tcgen05" and "128x128x64:tcgen05"), and for the grouped routes a
 * third, "128x128x64:tcgen05:splitk" (decode); a null or empty name lets the library choose by problem size, an
 * unknown name logs a decline and runs that default. */
int32_t quactlize_ppu_list_configs(quactlize_ppu_config_v1 const** configs);
int32_t quactlize_ppu_list_grouped_configs(quactlize_ppu_config_v1 const** configs);
int32_t quactlize_ppu_list_valid_dense_lowbit_configs_v2(quactlize_ppu_config_v2* configs, int32_t capacity, int m, int n,
                                                         int k, int group_size, int qtype);
int32_t quactlize_ppu_list_valid_dense_fully_quantized_configs_v2(quactlize_ppu_config_v2* configs, int32_t capacity, int m,
                                                                  int n, int k, int group_size, int qtype);
int32_t quactlize_ppu_list_valid_grouped_fully_quantized_configs_v2(quactlize_ppu_config_v2* configs, int32_t capacity,
                                                                    int total_rows, int n, int k, int group_size, int experts,
                                                                    int max_rows, int qtype);
int32_t quactlize_ppu_dense_lowbit_config_valid_v1(int m, int n, int k, int group_size, int qtype, char const* config_name);
int32_t quactlize_ppu_dense_fully_quantized_config_valid_v1(int m, int n, int k, int group_size, int qtype, char const* config_name);
int32_t quactlize_ppu_grouped_lowbit_config_valid_v1(int total_rows, int n, int k, int group_size, int experts, int max_rows,
                                                     int qtype, char const* config_name);
int32_t quactlize_ppu_grouped_fully_quantized_config_valid_v1(int total_rows, int n, int k, int group_size, int experts,
                                                              int max_rows, int qtype, char const* config_name);

/* Dense scale-first GEMM, D fp16 [m][n] = A fp16 [m][k] * W^T; W = cvt(u)*scale + zero with the reference converter's
 * convention cvt(u) = u - 8 for the int4-low formats (Q4_K/Q5_K/Q6_K) and u for Q2_K/Q3_K.
 * ppu_dense_backend.cu:666-734. */
int quactlize_ppu_dense_lowbit(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                               uint16_t const* zero, uint16_t* out, int m, int n, int k, int group_size, int qtype);
int quactlize_ppu_dense_lowbit_config_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                         uint16_t const* zero, uint16_t* out, int m, int n, int k, int group_size, int qtype,
                                         char const* config_name);
/* Dense fully-quantized GEMM (planes + packed units).  ppu_dense_backend.cu:741-846, quactlize_ppu_device.h:34-45.
 * The workspace (size from the query) receives the fp16 scale/zero planes derived from the units. */
int quactlize_ppu_dense_fully_quantized(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint8_t const* units,
                                        uint16_t* out, int m, int n, int k, int qtype);
int quactlize_ppu_dense_fully_quantized_config_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                  uint8_t const* units, uint16_t* out, int m, int n, int k, int qtype,
                                                  char const* config_name);
int64_t quactlize_ppu_dense_fully_quantized_workspace_bytes_v1(int m, int n, int k, int qtype);
int quactlize_ppu_dense_fully_quantized_dev_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                               uint8_t const* units, uint16_t* out, int m, int n, int k, int qtype,
                                               void* workspace, int64_t workspace_bytes, void* stream);
int quactlize_ppu_dense_fully_quantized_dev_v2(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                               uint8_t const* units, uint16_t* out, int m, int n, int k, int qtype,
                                               void* workspace, int64_t workspace_bytes, void* stream, char const* config_name);
/* Grouped scale-first GEMM, scale only: W = (u - 2^(W-1))*scale for two-plane formats, (u - 8)*scale for int4, u*scale
 * for int2.  Host entries take rows_per_expert [E]; device entries cumulative offsets [E+1].
 * ppu_dense_backend.cu:974-1127, quactlize_ppu_device.h:47-62. */
int quactlize_ppu_grouped_lowbit(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                 int const* rows_per_expert, uint16_t* out, int total_rows, int n, int k, int group_size,
                                 int experts, int qtype);
int quactlize_ppu_grouped_lowbit_config_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                           int const* rows_per_expert, uint16_t* out, int total_rows, int n, int k,
                                           int group_size, int experts, int qtype, char const* config_name);
int64_t quactlize_ppu_grouped_lowbit_workspace_bytes_v1(int max_rows, int n, int k, int group_size, int experts, int qtype);
int quactlize_ppu_grouped_lowbit_dev_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                        int const* offsets, uint16_t* out, int total_rows, int n, int k, int group_size,
                                        int experts, int max_rows, int qtype, void* workspace, int64_t workspace_bytes,
                                        void* stream);
int quactlize_ppu_grouped_lowbit_dev_v2(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                        int const* offsets, uint16_t* out, int total_rows, int n, int k, int group_size,
                                        int experts, int max_rows, int qtype, void* workspace, int64_t workspace_bytes,
                                        void* stream, char const* config_name);
/* Grouped fully-quantized GEMM.  ppu_dense_backend.cu:1134-1251, quactlize_ppu_device.h:64-77. */
int quactlize_ppu_grouped_fully_quantized(uint16_t const* act, uint8_t const* low, uint8_t const* high, uint8_t const* units,
                                          int const* rows_per_expert, uint16_t* out, int total_rows, int n, int k, int experts,
                                          int qtype);
int quactlize_ppu_grouped_fully_quantized_config_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                    uint8_t const* units, int const* rows_per_expert, uint16_t* out,
                                                    int total_rows, int n, int k, int experts, int qtype, char const* config_name);
int64_t quactlize_ppu_grouped_fully_quantized_workspace_bytes_v1(int max_rows, int n, int k, int experts, int qtype);
int quactlize_ppu_grouped_fully_quantized_dev_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                 uint8_t const* units, int const* offsets, uint16_t* out, int total_rows, int n,
                                                 int k, int experts, int max_rows, int qtype, void* workspace,
                                                 int64_t workspace_bytes, void* stream);
int quactlize_ppu_grouped_fully_quantized_dev_v2(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                 uint8_t const* units, int const* offsets, uint16_t* out, int total_rows, int n,
                                                 int k, int experts, int max_rows, int qtype, void* workspace,
                                                 int64_t workspace_bytes, void* stream, char const* config_name);
/* additive: generic per-group plane GEMM, dense (experts == 0) or grouped; W = (lo + 2^bits_lo*hi + code_offset)*scale + zero
 * (zero may be NULL); act_dtype 0 = fp16, 1 = bf16, output in the activation dtype; n % 128 == 0, k % 256 == 0.  The reference
 * reaches these shapes only through C++ templates (quactlize/include/moe_grouped_ppu.cuh:363-411). */
int quactlize_b200_gemm_plane_dev_v1(void const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                     uint16_t const* zero, void* out, int total_rows, int n, int k, int bits_lo, int bits_hi,
                                     int group_size, int code_offset, int act_dtype, int experts, int const* offsets, void* stream);

/* additive: v1 with an OUTPUT ROW MAP.  When out_rows is non-null it is a device array [total_rows] of addresses and
 * output row r (n elements) is stored at out_rows[r] instead of out + r*n (`out` may then be null).  In a grouped launch
 * total_rows may be an upper bound (the capacity of `act`); rows past offsets[experts] are never read or written. */
int quactlize_b200_gemm_plane_dev_v2(void const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                     uint16_t const* zero, void* out, int total_rows, int n, int k, int bits_lo, int bits_hi,
                                     int group_size, int code_offset, int act_dtype, int experts, int const* offsets,
                                     unsigned long long const* out_rows, void* stream);

/* additive: the split-K form of the plane GEMM for decode-sized (grouped) problems -- the B200 counterpart of the
 * reference's split-K grouped kernel, where slice z of K writes its own D plane and a light reduce follows
 * (quactlize/include/ppu_aiu_gemm_mixed_input_group.hpp:120-131,289-309).  128 x 128 tiles with shallow rings (several
 * CTAs per SM), K split over `splits` slices of whole 128-k pieces (0 = chosen so the grid fills the SMs, at most 8),
 * fp32 partial planes [splits][total_rows][n] in the caller's 16-byte aligned workspace, summed in slice order by a
 * second small kernel.  37 = workspace too small (size it with the query; splits 0 asks for the 8-slice maximum).
 * The grouped tactic name "128x128x64:tcgen05:splitk" selects the same form through the reference's *_dev_v2 entries
 * when their workspace (sized by their own queries) has room for the partial planes. */
int64_t quactlize_b200_gemm_plane_splitk_workspace_bytes_v1(int total_rows, int n, int splits);
int quactlize_b200_gemm_plane_splitk_dev_v1(void const* act, uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                            uint16_t const* zero, void* out, int total_rows, int n, int k, int bits_lo,
                                            int bits_hi, int group_size, int code_offset, int act_dtype, int experts,
                                            int const* offsets, int splits, void* workspace, int64_t workspace_bytes,
                                            void* stream);

/* No counterpart in the reference.  The fully-quantized dense GEMM of quactlize_ppu_dense_fully_quantized_dev_v1 for
 * callers that cannot allocate device memory and have no workspace to hand over: the fp16 scale/zero planes derived
 * from the packed units go to a fixed array inside the library's device image, QUACTLIZE_B200_STATIC_SCRATCH_BYTES
 * per device (held by every process that loads the library, on every device it uses, until exit, called or not).
 * Enqueues on `stream` and returns; allocates nothing.  37 = the planes (4 * k/group_size * n bytes) exceed
 * the array; 30 / 33 / 41 as for the regular entry.  The first call on a device looks the array's address up: make it
 * outside stream capture.  All calls on a device share the array (each rewrites what it reads, nothing needs
 * clearing); calls that may overlap in time on one device race on it. */
#define QUACTLIZE_B200_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)
int quactlize_b200_dense_fully_quantized_static_v1(uint16_t const* act, uint8_t const* low, uint8_t const* high,
                                                   uint8_t const* units, uint16_t* out, int m, int n, int k, int qtype,
                                                   void* stream);

/* additive: the reference's host ops gguf_unpack and gguf_*_artifact_dequantize (quactlize/csrc/preprocess/thop/
 * gguf_prepass_ops.cpp:767-799, 1118-1205) as device kernels, bit-exact with their host definitions.
 * unpack: raw blocks -> codes int8 [count][256] (signed for Q3_K/Q6_K), scale/zero fp16 [count][groups], W = code*scale+zero.
 * planes_dequantize: Native planes + fp16 planes [E][k/gs][n] -> fp16 [E][n][k] = half(float(u+code_shift)*scale + zero);
 * zero may be null; k % 8 == 0.  Both enqueue on `stream`, allocate nothing, return 0 = enqueued. */
int quactlize_b200_unpack_dev_v1(uint8_t const* blocks, int64_t block_bytes, int8_t* codes, uint16_t* scale, uint16_t* zero,
                                 int count, int qtype, void* stream);
int quactlize_b200_planes_dequantize_dev_v1(uint8_t const* low, uint8_t const* high, uint16_t const* scale,
                                            uint16_t const* zero, uint16_t* out, int experts, int n, int k, int bits_lo,
                                            int bits_hi, int group_size, int code_shift, void* stream);

/* ================================ expert parallelism over the GPUs of one node ================================== */

/* No counterpart in the reference (it has no multi-device code).  One process per GPU.  peer_alloc: a zeroed device
 * buffer from the runtime allocator plus its 64-byte IPC handle; peer_open / peer_close: map / unmap another rank's buffer
 * (NVLink peer access); peer_free.  These allocate and synchronise: set-up time only.
 * ep_count: routes per expert (expert ids int64 [routes]) -> counts int32 [experts].  ep_plan: with every rank's counts
 * [world][experts] (the caller all-gathers them), one CTA assigns every route of this rank an ITEM number in expert
 * order and writes, per item, the local token (route / top_k), the owner rank and the row in the owner's expert-major
 * receive buffer (experts in order, sources in rank order inside an expert); per route its item; and local_off
 * [experts/world + 1], the cumulative rows per local expert this rank's grouped GEMMs read as offsets.
 * ep_dispatch: item i (row item_token[i] of act, row_bytes long, a multiple of 16) is stored at row item_pos[i] of
 * peer_rows[item_rank[i]] and the tag (my_rank << 32 | i) at the same index of peer_tag[...]; the pointer tables are
 * device arrays of this process's mappings.  Plain peer stores; the caller orders them against the owner's reads with a
 * stream-ordered collective.  ep_return_addr: the owner turns received tags into addresses inside ITS mappings of the
 * senders' combine buffers (peer_comb[src] + item*row_bytes) for the row map of quactlize_b200_gemm_plane_dev_v2.
 * ep_combine: out[t] = sum_j weights[t][j] * comb[item_of_route[t*top_k+j]] (fp32, route order), bf16 rows of h elements.
 * silu_mul: out[r][c] = silu(gate_up[r][c]) * gate_up[r][f+c], bf16, for min(*rows_dev, max_rows) rows.
 * ep_sync: a rendezvous of the ranks through peer memory instead of a collective.  Every rank allocates a sync area of
 * ep_sync_bytes(world, experts) bytes (zeroed once), peers map it, peer_sync[w] is rank w's area.  One launch per rank
 * and barrier id (0..2): optionally stores counts_local[experts] into every rank's table counts_all[world][experts]
 * (byte 1024 of the area), then posts an epoch to every rank and waits (bounded, 2 s, status word on expiry) until
 * every rank's epoch has arrived.  Stream-ordered after the rank's earlier stores into peer memory. */
int quactlize_b200_peer_alloc(long long bytes, void** ptr, unsigned char* handle64);
int quactlize_b200_peer_open(unsigned char const* handle64, void** ptr);
int quactlize_b200_peer_close(void* ptr);
int quactlize_b200_peer_free(void* ptr);
int quactlize_b200_ep_count_dev_v1(long long const* expert_of_route, int routes, int experts, int* counts, void* stream);
int quactlize_b200_ep_plan_dev_v1(long long const* expert_of_route, int const* counts_all, int rank, int world, int experts, int routes,
                                  int top_k, int* item_token, int* item_rank, int* item_pos, int* item_of_route, int* local_off,
                                  void* stream);
int quactlize_b200_ep_dispatch_dev_v1(void const* act, int const* item_token, int const* item_rank, int const* item_pos,
                                      unsigned long long const* peer_rows, unsigned long long const* peer_tag, int my_rank,
                                      int items, int row_bytes, void* stream);
int quactlize_b200_ep_return_addr_dev_v1(unsigned long long const* tags, unsigned long long const* peer_comb, int world,
                                         int const* rows_dev, int max_rows, int row_bytes, unsigned long long* addr, void* stream);
int quactlize_b200_ep_combine_dev_v1(void const* comb, int const* item_of_route, float const* weights, void* out, int tokens,
                                     int top_k, int h, void* stream);
int quactlize_b200_silu_mul_dev_v1(void const* gate_up, void* out, int const* rows_dev, int max_rows, int f, void* stream);
int quactlize_b200_ep_sync_bytes(int world, int experts);
int quactlize_b200_ep_sync_dev_v1(unsigned long long const* peer_sync, int rank, int world, int id, int const* counts_local,
                                  int experts, void* stream);

/* ================================ host-only artifact producers ================================================== */

/* quactlize/include/quactlize_ppu_packed.h:12-33, quactlize/csrc/device/ppu_unit_pack.cpp:186-233 */
int64_t quactlize_ppu_units_bytes(int n, int k, int qtype);
int quactlize_ppu_prepare_units(uint8_t const* blocks, uint8_t* units, int n, int k, int qtype);
int quactlize_ppu_prepare_units_grouped(uint8_t const* blocks, uint8_t* units, int n, int k, int experts, int qtype);
int quactlize_ppu_prepare_fully_quantized_v1(uint8_t const* blocks, uint8_t* low, uint8_t* high, uint8_t* units, int n,
                                             int k, int experts, int qtype);
int quactlize_ppu_recover_fully_quantized_v1(uint8_t const* low, uint8_t const* high, uint8_t const* units,
                                             uint8_t* recovered, int n, int k, int experts, int qtype);
/* Plane placement for the tensor-core consumers.  This library's placement is the Native order, so these are
 * byte-identical copies.  quactlize/csrc/device/ppu_dense_layout.cu:108-208, ppu_backend.h:62-78. */
int quactlize_ppu_prepare_dense(uint8_t const* low_native, uint8_t const* high_native, uint8_t* low_layout,
                                uint8_t* high_layout, int n, int k, int qtype);
int quactlize_ppu_recover_dense(uint8_t const* low_layout, uint8_t const* high_layout, uint8_t* low_native,
                                uint8_t* high_native, int n, int k, int qtype);
int quactlize_ppu_prepare_dense_for_tile(uint8_t const* low_native, uint8_t const* high_native, uint8_t* low_layout,
                                         uint8_t* high_layout, int n, int k, int qtype, int tile_k);
int quactlize_ppu_recover_dense_for_tile(uint8_t const* low_layout, uint8_t const* high_layout, uint8_t* low_native,
                                         uint8_t* high_native, int n, int k, int qtype, int tile_k);
/* additive: the scale-first artifact producer (raw -> low, high, fp16 scale, fp16 zero), which the reference keeps in
 * its torch extension (quactlize/csrc/preprocess/thop/gguf_prepass_ops.cpp:809-878); any n > 0. */
int quactlize_b200_prepare_gemv(uint8_t const* blocks, uint8_t* low, uint8_t* high, uint16_t* scale, uint16_t* zero,
                                int n, int k, int experts, int qtype);
/* additive: packed-unit producer without the n % 256 restriction of the GEMM-facing entries. */
int quactlize_b200_pack_units(uint8_t const* blocks, uint8_t* units, int n, int k, int experts, int qtype);

/* additive: planes placed by the reference's device library (its "xplane" order: 64-column x TileK tiles, a bit
 * permutation inside each tile, quactlize/include/gguf_bc_vecdot.hpp:34-95) to and from the Native order this library's
 * kernels read.  One expert per call; n % 64 == 0, k % 256 == 0.  `slot` is the placed code index of logical (n, k). */
int quactlize_b200_xplane_to_native(uint8_t const* low_placed, uint8_t const* high_placed, uint8_t* low_native,
                                    uint8_t* high_native, int n, int k, int qtype);
int quactlize_b200_native_to_xplane(uint8_t const* low_native, uint8_t const* high_native, uint8_t* low_placed,
                                    uint8_t* high_placed, int n, int k, int qtype);
long long quactlize_b200_xplane_slot(int qtype, int high, int n, int k, int num_cols);

/* ================================ runtime ======================================================================= */

/* additive: make the NEXT runtime call of the given kind fail on the host (1 alloc, 2 H2D, 3 D2H, 4 sync, 6 launch);
 * the thread's latched status; read-and-clear of the device wait-status word (0 ok, 41 a bounded wait gave up).
 * Mirrors the reference's injectable fake runtime, quactlize/include/gemv_lowbit/gemv_rt.hpp:50-91. */
void quactlize_b200_rt_fail_next(int kind);
/* additive: release the device temporaries the calling thread's host-pointer entries keep parked for reuse. */
void quactlize_b200_rt_trim(void);
int quactlize_b200_rt_last_status(void);
int quactlize_b200_device_wait_status(void);
/* additive, for tests of the failure path: enqueue a one-CTA kernel that waits on an mbarrier nothing arms and gives
 * up after limit_ns (1 .. 100 000 000).  The kernel returns normally; the next quactlize_b200_device_wait_status()
 * reports 41 once, then 0.  No counterpart in the reference (its waits are unbounded). */
int quactlize_b200_debug_wait_probe(long long limit_ns, void* stream);
/* additive, for tests: how many launches of the swapped tensor-core form (weights converted into tensor memory as the A
 * operand; opt-in through QUACTLIZE_B200_GEMM_SWAP) this process has enqueued.  No counterpart in the reference. */
long long quactlize_b200_debug_gemm_swap_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* QUACTLIZE_B200_H_ */
