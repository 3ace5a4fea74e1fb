"""Generates ``philox_kat.json``: Philox4x32-10 known answers from an implementation that
is independent of this repository -- ATen's ``at::philox_engine`` header that ships with
the installed torch -- by compiling and running a few lines of C++ against it.

In that engine the 128-bit counter is (offset lo, offset hi, subsequence lo, subsequence hi)
and the key is (seed lo, seed hi); the first four outputs of a fresh engine are the Philox
block of that counter. Run: ``python tests/golden/make_philox_kat.py``.
"""
import json
import os
import subprocess
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
SRC = r"""
#include <ATen/core/PhiloxRNGEngine.h>
#include <cstdio>
#include <cstdint>
int main() {
  const uint64_t seeds[] = {0ull, 1ull, 0x123456789abcdef0ull, 0xffffffffffffffffull, 20241125ull};
  const uint64_t subs[]  = {0ull, 1ull, 0x00000001ffffffffull, 0xdeadbeefcafef00dull};
  const uint64_t offs[]  = {0ull, 1ull, 79ull, 0x0000000500000013ull, 0xffffffff00000000ull};
  bool first = true;
  std::printf("[");
  for (uint64_t seed : seeds) for (uint64_t sub : subs) for (uint64_t off : offs) {
    at::philox_engine eng(seed, sub, 0);
    eng.set_offset(off);
    uint32_t o[4];
    for (int i = 0; i < 4; i++) o[i] = eng();
    std::printf("%s{\"counter\":[%u,%u,%u,%u],\"key\":[%u,%u],\"out\":[%u,%u,%u,%u]}",
                first ? "" : ",\n",
                (uint32_t)off, (uint32_t)(off >> 32), (uint32_t)sub, (uint32_t)(sub >> 32),
                (uint32_t)seed, (uint32_t)(seed >> 32), o[0], o[1], o[2], o[3]);
    first = false;
  }
  std::printf("]\n");
  return 0;
}
"""


def main():
    inc = os.path.join(os.path.dirname(torch.__file__), "include")
    with tempfile.TemporaryDirectory() as td:
        src = Path(td) / "kat.cpp"
        exe = Path(td) / "kat"
        src.write_text(SRC)
        subprocess.run(["g++", "-std=c++17", "-O1", f"-I{inc}", "-o", str(exe), str(src)], check=True)
        out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    vecs = json.loads(out)
    doc = {"source": f"at::philox_engine, torch {torch.__version__}", "vectors": vecs}
    lines = ",\n".join(json.dumps(v, separators=(",", ":")) for v in vecs)
    (HERE / "philox_kat.json").write_text(
        '{"source": %s,\n"vectors": [\n%s\n]}\n' % (json.dumps(doc["source"]), lines))
    print(f"wrote {len(vecs)} vectors")


if __name__ == "__main__":
    main()
