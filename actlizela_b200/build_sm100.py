#!/usr/bin/env python3
"""Build the native cuda_sm100 library in-tree and write its receipt.

    python -m actlizela_b200.build_sm100 [--out DIR] [--compiler NVCC] [--verbose-ptxas]

One nvcc invocation compiles every kernel for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and links ``libactlize_la_sm100.so``.  The static
shape table ``sm100_policy.json`` is rendered into a C++ include so that the native
``actlize_la_sm100_select`` and the Python selector share one source.  ``build.json`` records
the compiler, flags and SHA-256 of every source and of the library; the loader refuses a
library whose hash differs.  Same role as the reference's tools/build_gdn_sm90.py:28-197
(device compile with the 90a gencode, receipt with source/compiler hashes), without the
Torch-extension link step because the boundary here is a plain C ABI.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
from pathlib import Path
import shlex
import subprocess
import sys

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
SOURCE = PACKAGE / "csrc" / "backends" / "sm100"
INCLUDE = ROOT / "include"
UNITS = ("abi.cu", "gdn_simt.cu", "gdn_umma.cu", "gdn_aux.cu", "out_proj.cu", "static_scratch.cu")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
         "-DNDEBUG", *ARCH_FLAGS]


def sha(path):
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


def render_policy_table(policy_path, out_path):
    data = json.loads(Path(policy_path).read_text())
    ids = data["configuration_ids"]
    rows = ",\n".join(
        "  {%d, %d, %d, %d, %d, %d, %d}" % (*row["shape"], ids[row["configuration"]], int(row.get("segments", 1)),
                                             int(row.get("parallel", 1)))
        for row in data["rows"])
    out_path.write_text(
        "// generated from sm100_policy.json (%s); do not edit\n"
        "struct PolicyRow { int b, t, hk, hv, config, segments, parallel; };\n"
        "constexpr int kPolicyDefault = %d;\n"
        "constexpr PolicyRow kPolicyRows[] = {\n%s\n};\n"
        % (data["id"], ids[data["default"]], rows))


def build(out=None, compiler=None, verbose_ptxas=False, quiet=False, defines=()):
    out = Path(out) if out else PACKAGE / "_native"
    out.mkdir(parents=True, exist_ok=True)
    generated = out / "generated"
    generated.mkdir(exist_ok=True)
    compiler = Path(compiler or Path(os.getenv("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc")
    if not compiler.is_file():
        raise RuntimeError(f"compiler missing: {compiler}")
    policy_path = PACKAGE / "sm100_policy.json"
    render_policy_table(policy_path, generated / "sm100_policy_table.inc")
    sources = sorted(p for p in SOURCE.iterdir() if p.suffix in (".cu", ".cuh", ".h"))
    identity = dict(
        target="cuda_sm100", arch="sm_100a", abi_version=1, complete=False,
        compiler=str(compiler),
        compiler_version=subprocess.check_output([str(compiler), "--version"], text=True).strip().splitlines()[-1],
        flags=[*FLAGS, *(f"-D{d}" for d in defines)], policy_sha256=sha(policy_path),
        source_sha256={str(p.relative_to(ROOT)): sha(p) for p in [*sources, INCLUDE / "actlize_la_sm100.h"]})
    receipt = out / "build.json"
    receipt.write_text(json.dumps(identity, indent=2) + "\n")
    library = out / "libactlize_la_sm100.so"
    command = [str(compiler), *identity["flags"], "-shared", f"-I{INCLUDE}", f"-I{SOURCE}", f"-I{generated}",
               *(["-Xptxas", "-v"] if verbose_ptxas else []),
               *(str(SOURCE / unit) for unit in UNITS), "-o", str(library)]
    if not quiet:
        print("[sm100 build]", shlex.join(command), flush=True)
    log = out / "build.log"
    with log.open("w") as stream:
        stream.write(shlex.join(command) + "\n")
        stream.flush()
        result = subprocess.run(command, stdout=stream, stderr=subprocess.STDOUT)
    if result.returncode:
        sys.stderr.write(log.read_text()[-6000:])
        raise RuntimeError(f"nvcc failed rc={result.returncode}; see {log}")
    after = {str(p.relative_to(ROOT)): sha(p) for p in [*sources, INCLUDE / "actlize_la_sm100.h"]}
    if after != identity["source_sha256"]:
        raise RuntimeError("source changed during build; do not use this binary")
    identity.update(library=library.name, library_sha256=sha(library), complete=True)
    receipt.write_text(json.dumps(identity, indent=2) + "\n")
    if not quiet:
        print(f"[sm100 build] PASS scope=COMPILE_LINK_ONLY library={library} device=NOT_RUN")
    return library


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--out", type=Path)
    ap.add_argument("--compiler", type=Path)
    ap.add_argument("--verbose-ptxas", action="store_true")
    ap.add_argument("--define", action="append", default=[], help="extra -D macro (diagnostic builds)")
    args = ap.parse_args()
    build(args.out, args.compiler, args.verbose_ptxas, defines=args.define)
    if args.verbose_ptxas:
        print((Path(args.out or PACKAGE / "_native") / "build.log").read_text())


if __name__ == "__main__":
    main()
