"""Test infrastructure: builds the 32-bit residual-stream kernel files (lp_linear.cu, lp_stream32.cu, lp_seqmix.cu, lp_winattn.cu, lp_mingru.cu, lp_mlstm.cu, lp_moe.cu — kernels
AND their host entry points) for the CPU emulator: includes dropped, dynamic shared memory turned into a static buffer, launches
rewritten (launch_rewrite.py), runtime names from host_emu.h.  The result exports the same C symbols as the native library."""
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
SOURCES = ("lp_linear", "lp_stream32", "lp_seqmix", "lp_winattn", "lp_mingru", "lp_mlstm", "lp_moe")


def build_emulated(out: Path) -> Path:
    sys.path.insert(0, str(ROOT / "tests/emu"))
    from launch_rewrite import rewrite_launches
    out.mkdir(parents=True, exist_ok=True)
    units = []
    for name in SOURCES:
        src = (ROOT / "leopard_b200/csrc" / f"{name}.cu").read_text()
        for line in ('#include "lp_host.h"\n', '#include "../../include/leopard_b200.h"\n'):
            assert line in src, (name, line)
            src = src.replace(line, "")
        src = src.replace("  extern __shared__ float dyn_smem[];", "  static float dyn_smem[1 << 16];")
        assert "extern __shared__" not in src and "asm" not in src, name
        src = rewrite_launches(src)
        assert "<<<" not in src, name
        (out / f"{name}_src.inc").write_text(src)
        unit = out / f"{name}_emu.cpp"
        unit.write_text('#include "host_emu.h"\n#include "leopard_b200.h"\n'
                        f'#include "{name}_src.inc"\n')
        units.append(str(unit))
    (out / "common_emu.cpp").write_text(
        '#include "host_emu.h"\nextern "C" {\nconst char* lp_last_error(void) { return lp::g_emu_err; }\n'
        'long long lp_launch_count(void) { return 0; }\nint lp_abi_version(void) { return 3; }\n}\n')
    lib = out / "libstream32_emu.so"
    r = subprocess.run(["g++", "-std=c++20", "-O2", "-pthread", "-shared", "-fPIC", "-ffp-contract=off", "-fno-strict-aliasing", "-I", str(out),
                        "-I", str(ROOT / "tests/emu"), "-I", str(ROOT / "include"), *units, str(out / "common_emu.cpp"), "-o", str(lib)],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(r.stderr[-6000:])
    return lib
