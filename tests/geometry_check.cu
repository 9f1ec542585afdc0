// Host-side check of the index arithmetic that the lane-group kernels share (reduce_seg_group_kernel,
// seg_group_fwd/bwd_kernel, argmax_group_kernel): for every run length, array alignment and run
// number, the (pack, lane, element) walk chosen by kn::group_geometry must visit every element of the
// run exactly once (so nothing outside it either) and take 16-byte accesses only at 16-byte aligned
// addresses.  Also the tiling invariants of kn::rows_geometry.  Runs on the CPU (the device
// query falls back to 148 SMs); prints "cases N bad M".
#include <cstdio>
#include <vector>

#include "reduce.cuh"

using namespace kn;

template <typename T>
static void check_groups(long& cases, long& bad) {
  constexpr uint32_t VEC = VecN<T>::value;
  std::vector<int> cover;
  for (uint32_t D = 1; D <= 2100; D += (D < 300 ? 1 : 7)) {
    for (uint32_t a0 = 0; a0 < VEC; a0++) {                       // offset of the array inside a 16-byte line
      const uintptr_t array = 4096 + a0 * sizeof(T);
      const GroupGeom g = group_geometry<T>((const void*)array, D, 16);
      const bool may_be_off = !(a0 == 0 && D % VEC == 0);
      const uint64_t packs_needed = ((uint64_t)D + (may_be_off ? VEC - 1 : 0) + VEC - 1) / VEC;
      cases++;
      if (g.np == 0) {
        if (packs_needed <= 512) { bad++; std::printf("no geometry for D=%u a0=%u\n", D, a0); }
        continue;
      }
      if ((uint64_t)g.g * g.np < packs_needed) { bad++; std::printf("too small D=%u a0=%u\n", D, a0); continue; }
      for (uint32_t seg = 0; seg < 2 * VEC + 1; seg++) {          // runs start at every offset the layout can give
        const uintptr_t p = array + (uintptr_t)seg * D * sizeof(T);
        const uint32_t mis = (uint32_t)((p & 15u) / sizeof(T));
        const uint32_t total = mis + D;
        cover.assign(D, 0);
        bool unaligned = false;
        for (int j = 0; j < g.np; j++)
          for (int lane = 0; lane < g.g; lane++) {
            const uint32_t e0 = ((uint32_t)j * g.g + lane) * VEC;
            if (e0 >= mis && e0 + VEC <= total) {
              if (((p - mis * sizeof(T)) + e0 * sizeof(T)) % 16 != 0) unaligned = true;
              for (uint32_t e = 0; e < VEC; e++) cover[e0 + e - mis]++;
            } else {
              for (uint32_t e = 0; e < VEC; e++) {
                const uint32_t i = e0 + e;
                if (i >= mis && i < total) cover[i - mis]++;
              }
            }
          }
        bool once = true;
        for (uint32_t i = 0; i < D; i++) once &= cover[i] == 1;
        cases++;
        if (!once || unaligned) { bad++; std::printf("walk wrong: D=%u a0=%u seg=%u once=%d unaligned=%d\n", D, a0, seg, once, unaligned); }
      }
    }
  }
}

static void check_rows(long& cases, long& bad) {
  const uint32_t rows_set[] = {1, 7, 10, 31, 32, 33, 64, 100, 128, 1000, 1024, 2047, 2048, 4096, 5021, 8192, 50257, 1u << 20};
  const uint32_t cols_set[] = {1, 2, 63, 64, 255, 256, 1000, 4096, 8192, 100000, 524288};
  for (uint32_t rows : rows_set)
    for (uint32_t cols : cols_set)
      for (uint32_t nbatch : {1u, 3u, 1000u})
        for (uint32_t vec : {2u, 4u})
          for (int forced : {0, 1, 8})
            for (bool by_rv : {false, true}) {
              auto ok = [&](uint32_t rv) { return rows % rv == 0; };
              const RowsGeom g = rows_geometry(rows, cols, nbatch, vec, 8, ok, forced, by_rv);
              cases++;
              const bool rv_ok = (g.rv == 1 || g.rv == 2 || g.rv == 4) && g.rv <= vec && rows % g.rv == 0;
              const bool tiles_ok = (uint64_t)g.tiles * 32 * g.rv >= rows && (uint64_t)(g.tiles - 1) * 32 * g.rv < rows;
              const bool cs_ok = g.cs == 1 || g.cs == 2 || g.cs == 4 || g.cs == 8;
              if (!rv_ok || !tiles_ok || !cs_ok) { bad++; std::printf("rows geometry wrong: rows=%u cols=%u rv=%u tiles=%u cs=%u\n", rows, cols, g.rv, g.tiles, g.cs); }
            }
}

int main() {
  long cases = 0, bad = 0;
  check_groups<float>(cases, bad);
  check_groups<double>(cases, bad);
  check_rows(cases, bad);
  std::printf("cases %ld bad %ld\n", cases, bad);
  return bad != 0;
}
