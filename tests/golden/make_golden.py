#!/usr/bin/env python3
"""Makes tests/golden/lfm3_R_last_logits.f32: the reference project's own LFM3 code, on its CPU
backend in float32, run on the tiny random model R (tests/tiny.py: the reference's layout with
sandwich norms, a gate per head, partly rotated heads, a sliding layer, 7 taps).

    python tests/golden/make_golden.py --reference /path/to/xpu-serve [--build-dir DIR]

Steps: write model R with this repository's random-weights mode (float32, seed and scale factors
of tests/tiny.py); configure and build the reference's core and cpu-ref libraries with CMake
(no GPU backend); compile ref_logits.cpp against them; run it for the prompt lengths in LENGTHS.
Needs cmake, a C++20 compiler and OpenSSL headers; takes about a minute. The reference's sources
are only read and linked, never copied. tests/test_plain.py compares the plain implementation
with the file this writes.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]

LENGTHS = [1, 5, 13, 23, 40]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of v1k22/xpu-serve (it is configured with CMake, not changed)")
    ap.add_argument("--build-dir", default=None)
    args = ap.parse_args()
    import tiny
    build = args.build_dir or tempfile.mkdtemp(prefix="xs_ref_build_")
    os.makedirs(build, exist_ok=True)
    model = tiny.make_folder(os.path.join(build, "models"), "R", "float32")
    ref = os.path.abspath(args.reference)
    run = lambda cmd: subprocess.run(cmd, check=True)   # noqa: E731
    run(["cmake", "-S", ref, "-B", os.path.join(build, "cmake"), "-DXS_BUILD_TESTS=OFF", "-DCMAKE_BUILD_TYPE=Release"])
    run(["cmake", "--build", os.path.join(build, "cmake"), "--target", "xs_backends", "-j", str(os.cpu_count() or 4)])
    libs = []
    for dirpath, _, files in os.walk(os.path.join(build, "cmake")):
        libs += [os.path.join(dirpath, f) for f in files if f.endswith(".a")]
    exe = os.path.join(build, "ref_logits")
    inc = [f"-I{os.path.join(ref, 'src')}", f"-I{os.path.join(ref, 'third_party')}",
           f"-I{os.path.join(ref, 'third_party', 'nlohmann')}"]
    run(["g++", "-std=c++20", "-O2", *inc, os.path.join(HERE, "ref_logits.cpp"), "-o", exe,
         "-Wl,--start-group", *libs, "-Wl,--end-group", "-lpthread", "-lssl", "-lcrypto"])
    out = os.path.join(HERE, "lfm3_R_last_logits.f32")
    run([exe, model, out, *map(str, LENGTHS)])
    with open(os.path.join(HERE, "lfm3_R_last_logits.json"), "w") as f:
        json.dump({"config": "R", "seed": tiny.SEEDS["R"], "dtype": "float32", "lengths": LENGTHS,
                   "vocab": tiny.CONFIGS["R"]["vocab_size"], "made_by": "tests/golden/make_golden.py",
                   "reference_backend": "cpu-ref, float32"}, f, indent=1)
    print(f"wrote {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
