/* Test helper: a C99 reader of the shared-memory pair table that uses include/ks_pairtab_shm.h alone (no library).
 * usage: pairtab_reader <segment name> <min_gangs>; stdin: lines "shape_a shape_b type_a type_b" (decimal u64);
 * stdout: per line "eff_bits gangs kus_a_bits" (efficiency as the bits of the float, -1 -1 if there is no row). */
#include <fcntl.h>
#include <inttypes.h>
#include <stdio.h>
#include <stdlib.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "../include/ks_pairtab_shm.h"

int main(int argc, char** argv) {
  if (argc != 3) return 2;
  const int fd = shm_open(argv[1], O_RDONLY, 0);
  if (fd < 0) { perror("shm_open"); return 1; }
  struct stat st;
  if (fstat(fd, &st) != 0) return 1;
  const void* seg = mmap(NULL, (size_t)st.st_size, PROT_READ, MAP_SHARED, fd, 0);
  close(fd);
  if (seg == MAP_FAILED) return 1;
  const ks_pairtab_header* h = ks_pairtab_check(seg, (uint64_t)st.st_size);
  if (!h) { fprintf(stderr, "not a pair table\n"); return 1; }
  printf("%" PRIu64 " %" PRIu64 " %" PRIu64 " %" PRIu64 " %" PRIu64 "\n", h->generation, h->shape.n_keys, h->shape.n_rows, h->type.n_keys, h->type.n_rows);
  const uint32_t min_gangs = (uint32_t)strtoul(argv[2], NULL, 10);
  uint64_t sa, sb, ta, tb;
  while (scanf("%" SCNu64 " %" SCNu64 " %" SCNu64 " %" SCNu64, &sa, &sb, &ta, &tb) == 4) {
    const ks_pairtab_val* v = ks_pairtab_lookup_eff(seg, sa, sb, ta, tb, min_gangs);
    const double kus = ks_pairtab_kernel_us(seg, sa, ta);
    uint64_t kbits;
    memcpy(&kbits, &kus, 8);
    if (v) {
      uint32_t ebits;
      memcpy(&ebits, &v->efficiency, 4);
      printf("%" PRIu32 " %" PRIu32 " %" PRIu64 "\n", ebits, v->gangs, kbits);
    } else {
      printf("-1 -1 %" PRIu64 "\n", kbits);
    }
  }
  return 0;
}
