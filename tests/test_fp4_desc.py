"""The block-scaled FP4 MMA's instruction descriptor, held to CUTLASS's own encoder (no GPU needed): a small host program
is compiled against cute/arch/mma_sm100_desc.hpp - found through the installed flashinfer package, which vendors the
CUTLASS headers - and prints make_instr_desc_block_scaled's 32 bits for E2M1 x E2M1 under UE4M3 factors (NVFP4) and under
UE8M0 factors (MXFP4); the library's mm_fp4_desc must give the same words. Skipped where the headers or nvcc are missing."""
import importlib.util
import os
import shutil
import subprocess

import pytest

PROGRAM = r"""
#include <cstdio>
#include <cstdint>
#include <cute/arch/mma_sm100_desc.hpp>
using namespace cute;
template <class SF, int N> uint32_t desc(uint32_t sf_id) {
  UMMA::InstrDescriptorBlockScaled d = UMMA::make_instr_desc_block_scaled<float_e2m1_t, float_e2m1_t, float, SF, 128, N,
                                                                          UMMA::Major::K, UMMA::Major::K>();
  d.a_sf_id_ = sf_id, d.b_sf_id_ = sf_id;
  return (uint32_t) d;
}
int main() {
  printf("%u %u %u %u %u %u\n", desc<float_ue4m3_t, 128>(0), desc<float_ue4m3_t, 256>(0), desc<float_ue4m3_t, 16>(0),
         desc<float_ue8m0_t, 128>(0), desc<float_ue8m0_t, 256>(2), desc<float_ue8m0_t, 48>(2));
  return 0;
}
"""


def _cutlass_include():
    spec = importlib.util.find_spec("flashinfer")
    if not spec or not spec.submodule_search_locations:
        return None
    inc = os.path.join(list(spec.submodule_search_locations)[0], "data", "cutlass", "include")
    return inc if os.path.exists(os.path.join(inc, "cute", "arch", "mma_sm100_desc.hpp")) else None


def test_instruction_descriptor_equals_cutlass(tmp_path, lib):
    inc, nvcc = _cutlass_include(), shutil.which("nvcc")
    if not inc or not nvcc:
        pytest.skip("CUTLASS headers (through flashinfer) or nvcc not available")
    src, exe = tmp_path / "desc.cu", tmp_path / "desc"
    src.write_text(PROGRAM)
    build = subprocess.run([nvcc, "-std=c++17", "-I" + inc, "-o", str(exe), str(src)], capture_output=True, text=True)
    if build.returncode != 0:
        pytest.skip("the vendored CUTLASS headers do not compile as a host program here: " + build.stderr[-300:])
    want = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    got = [lib.mm_fp4_desc(0, 128, 0), lib.mm_fp4_desc(0, 256, 0), lib.mm_fp4_desc(0, 16, 0), lib.mm_fp4_desc(1, 128, 0),
           lib.mm_fp4_desc(1, 256, 2), lib.mm_fp4_desc(1, 48, 2)]
    assert got == want, (["%08x" % v for v in got], ["%08x" % v for v in want])


LAYOUT = r"""
#include <cstdio>
#include <cutlass/detail/sm100_blockscaled_layout.hpp>
using namespace cute;
int main() {
  typename cutlass::detail::Sm1xxBlockScaledBasicChunk<16>::SfKMajorAtom a16;
  typename cutlass::detail::Sm1xxBlockScaledBasicChunk<32>::SfKMajorAtom a32;
  int bad = 0;
  for (int m = 0; m < 128; m++)
    for (int f = 0; f < 4; f++) {
      const int mine = (m & 31) * 16 + (m >> 5) * 4 + f;  // row m's factor f in a 512-byte chunk
      bad += (int) a16(m, f * 16) != mine || (int) a16(m, f * 16 + 15) != mine || (int) a32(m, f * 32) != mine;
    }
  printf("%d %d\n", bad, (int) cosize(a16));
  return 0;
}
"""


def test_scale_factor_chunk_layout_equals_cutlass(tmp_path):
    """the scale factors' chunk layout (128 rows x 4 factors in 512 bytes: byte (r % 32) * 16 + (r / 32) * 4 + f), as the
    kernel's producers write it, against CUTLASS's Sm1xxBlockScaledBasicChunk atom"""
    inc, nvcc = _cutlass_include(), shutil.which("nvcc")
    if not inc or not nvcc:
        pytest.skip("CUTLASS headers (through flashinfer) or nvcc not available")
    src, exe = tmp_path / "layout.cu", tmp_path / "layout"
    src.write_text(LAYOUT)
    build = subprocess.run([nvcc, "-std=c++17", "-Wno-deprecated-gpu-targets", "-I" + inc, "-o", str(exe), str(src)], capture_output=True, text=True)
    if build.returncode != 0:
        pytest.skip("the vendored CUTLASS headers do not compile as a host program here: " + build.stderr[-300:])
    assert subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split() == ["0", "512"]
