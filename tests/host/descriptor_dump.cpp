// Host-only program: prints descriptor values computed by the library's own
// constexpr packers (ptx.jl_b200/csrc/sm100_prims.cuh) so that the Python test can
// compare them with independently written formulas and with the reference's
// known-answer constants.
#include <cstdio>
#include "sm100_prims.cuh"
#include "attn_tiles.cuh"

using namespace ptxb200;

int main() {
  printf("sdesc_b128 %llx\n", (unsigned long long)make_sdesc(0, 16, 1024, kLayoutB128));
  const unsigned addrs[] = {0u, 16u, 0x400u, 0x3FFF0u};
  const unsigned leads[] = {0u, 16u, 16384u, 0x12340u};
  const unsigned strides[] = {0u, 1024u, 0x2abc0u};
  const unsigned layouts[] = {0u, 1u, 2u, 4u, 6u};
  for (unsigned a : addrs) for (unsigned l : leads) for (unsigned s : strides) for (unsigned y : layouts)
    printf("sdesc %u %u %u %u %llx %x %x\n", a, l, s, y, (unsigned long long)make_sdesc(a, l, s, y),
           sdesc_lo(a, l), sdesc_hi(s, y));
  const unsigned ms[] = {64u, 128u, 256u};
  for (unsigned m : ms) for (unsigned n = 8; n <= 256; n += 8) for (int am = 0; am < 2; ++am) for (int bm = 0; bm < 2; ++bm)
    printf("idesc %u %u %d %d %x\n", m, n, am, bm, make_idesc_bf16_f32(m, n, am != 0, bm != 0));
  for (unsigned lane = 0; lane < 128; lane += 31) printf("tmem %u %x\n", lane, tmem_addr(0x00070000u, lane, 5));
  printf("attn128 %x %x %d %d %d\n", AttnTile<128>::kIdescQK, AttnTile<128>::kIdescPV, AttnTile<128>::kTileBytes,
         AttnTile<128>::kQKAtoms, AttnTile<128>::kPVAtoms);
  printf("attn64 %x %x %d %d %d\n", AttnTile<64>::kIdescQK, AttnTile<64>::kIdescPV, AttnTile<64>::kTileBytes,
         AttnTile<64>::kQKAtoms, AttnTile<64>::kPVAtoms);
  return 0;
}
