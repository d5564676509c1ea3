/* A C caller of the drop-in boundary: loads the library the way the reference's loader does (dlopen + dlsym of plain-C
 * symbols), and uses host-only entries.  Compiled and run by tests/test_abi_cpu.py; proves include/quactlize_b200.h is C. */
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "quactlize_b200.h"

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  void* h = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
  if (!h) { fprintf(stderr, "dlopen: %s\n", dlerror()); return 3; }
  int64_t (*units_bytes)(int, int, int) = (int64_t (*)(int, int, int))dlsym(h, "quactlize_ppu_units_bytes");
  int (*prepare_units)(uint8_t const*, uint8_t*, int, int, int) =
      (int (*)(uint8_t const*, uint8_t*, int, int, int))dlsym(h, "quactlize_ppu_prepare_units");
  int32_t (*list_configs)(quactlize_ppu_config_v1 const**) = (int32_t (*)(quactlize_ppu_config_v1 const**))dlsym(h, "quactlize_ppu_list_configs");
  int (*vecdot_dense)(uint8_t const*, int64_t, uint16_t const*, float*, int, int, int) =
      (int (*)(uint8_t const*, int64_t, uint16_t const*, float*, int, int, int))dlsym(h, "quactlize_ppu_vecdot_dense");
  if (!units_bytes || !prepare_units || !list_configs || !vecdot_dense) return 4;
  int const n = 256, k = 512, qtype = 12;
  int64_t const ub = units_bytes(n, k, qtype);
  if (ub != (int64_t)(k / 256) * n * 16) return 5;
  uint8_t* blocks = (uint8_t*)calloc((size_t)n * (k / 256), 144);
  uint8_t* units = (uint8_t*)malloc((size_t)ub);
  for (size_t i = 0; i < (size_t)n * (k / 256) * 144; ++i) blocks[i] = (uint8_t)(i * 73 + 7);
  if (prepare_units(blocks, units, n, k, qtype) != 0) return 6;
  /* the unit of (superblock 0, row 0) starts with the block's d and dmin */
  if (memcmp(units, blocks, 4) != 0) return 7;
  quactlize_ppu_config_v1 const* cfg = NULL;
  if (list_configs(&cfg) < 1 || !cfg || !cfg[0].name) return 8;
  /* argument refusals come back as codes, never as aborts */
  if (vecdot_dense(NULL, 144, NULL, NULL, n, k / 256, qtype) == 0) return 9;
  printf("ok %lld %s\n", (long long)ub, cfg[0].name);
  free(blocks); free(units);
  return 0;
}
