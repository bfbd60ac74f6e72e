"""In-tree build of every native artefact of the package.

Artefacts (all written next to the package so they travel with a checkout and are what the Python side
loads):

* ``fuselink_b200/_C.so``                    torch extension: sm_100a kernels, cuMem layer, monitor bindings
* ``fuselink_b200/lib/libnccl-net-fuselink.so``  the ncclNet plugin (``NCCL_NET_PLUGIN=fuselink``)
* ``fuselink_b200/lib/libfuselink.so``           kernels + cuMem regions + monitor as a C library (``include/fuselink.h``)
* ``fuselink_b200/lib/fuselink-monitor``      stand-alone monitor daemon
* ``fuselink_b200/lib/fl_net_harness``        two-process driver of the plugin vtable used by the CPU tests

CUDA sources are compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``); nvcc
cross-compiles without a GPU.  A content hash per object keeps rebuilds incremental.

Run ``python -m fuselink_b200.build`` (or ``build_all()``).
"""
from __future__ import annotations

import hashlib
import json
import os
import shlex
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "_build"
LIB = PKG / "lib"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-g", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"]

KERNELS = ["grouped_gemm", "comm_kernels", "embbag", "kv_pack", "moe_dispatch", "moe_dispatch_noalloc", "fp8_gemm", "shadow_reduce"]
NET_SRCS = ["plugin", "tcp_transport", "tcp_endpoints", "params", "conn_manager", "ib_transport", "nvl_channel", "logging", "rdma_transport", "soft_provider", "verbs_provider", "nic_rate"]


def _sha(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(set(paths)):
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _headers():
    return [p for p in CSRC.rglob("*") if p.suffix in (".h", ".cuh", ".hpp")]


def _run(cmd, verbose):
    if verbose:
        print("  $", " ".join(shlex.quote(str(c)) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed ({r.returncode}):\n{' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


class _Stamp:
    def __init__(self):
        self.path = OBJ / "stamps.json"
        try:
            self.data = json.loads(self.path.read_text())
        except Exception:
            self.data = {}

    def fresh(self, out: Path, key: str) -> bool:
        return out.exists() and self.data.get(str(out.relative_to(PKG))) == key

    def mark(self, out: Path, key: str):
        self.data[str(out.relative_to(PKG))] = key

    def save(self):
        OBJ.mkdir(exist_ok=True)
        self.path.write_text(json.dumps(self.data, indent=0, sort_keys=True))


def _torch_flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"], "-isystem", f"{CUDA_HOME}/include"]
    libdir = str(Path(torch.__file__).parent / "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    link = [f"-L{libdir}", f"-Wl,-rpath,{libdir}", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10", "-lc10_cuda",
            "-ltorch_cuda", f"-L{CUDA_HOME}/lib64", f"-Wl,-rpath,{CUDA_HOME}/lib64", "-lcudart", "-ldl", "-lrt", "-lpthread"]
    return inc, defs, link


def build_all(verbose: bool = False, jobs: int | None = None) -> dict:
    """Compile everything that is out of date.  Returns {artefact: path}."""
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    stamp = _Stamp()
    hdrs = _headers()
    jobs = jobs or min(8, os.cpu_count() or 4)
    tasks = []  # (out, cmd, key)

    def add(out: Path, srcs, cmd, extra=""):
        key = _sha(list(srcs) + hdrs, extra + " ".join(map(str, cmd)))
        if not stamp.fresh(out, key):
            tasks.append((out, cmd, key))
        return out

    # ---- CUDA kernels --------------------------------------------------------------------------
    cu_objs = []
    for k in KERNELS:
        src = CSRC / "kernels" / f"{k}.cu"
        if not src.exists():
            continue
        out = OBJ / f"{k}.o"
        cu_objs.append(add(out, [src], [NVCC, *NVCC_FLAGS, "-Xptxas", "-v", "-c", src, "-o", out]))

    # ---- host C++ shared by the extension and the plugin -----------------------------------------
    host_objs = []
    for rel in ["mem/vmm.cc", "monitor/monitor.cc"]:
        src = CSRC / rel
        out = OBJ / (Path(rel).stem + ".o")
        host_objs.append(add(out, [src], [CXX, *CXX_FLAGS, f"-I{CUDA_HOME}/include", "-c", src, "-o", out]))

    # ---- torch extension ------------------------------------------------------------------------
    inc, defs, tlink = _torch_flags()
    ext_objs = []
    for rel in ["torch/bindings.cpp", "monitor/monitor_py.cpp"]:
        src = CSRC / rel
        out = OBJ / (Path(rel).stem + ".o")
        ext_objs.append(add(out, [src], [CXX, *CXX_FLAGS, *defs, *inc, "-c", src, "-o", out]))

    # ---- plugin objects ---------------------------------------------------------------------------
    net_objs = []
    for n in NET_SRCS:
        src = CSRC / "net" / f"{n}.cc"
        if not src.exists():
            continue
        out = OBJ / f"net_{n}.o"
        net_objs.append(add(out, [src], [CXX, *CXX_FLAGS, f"-I{CUDA_HOME}/include", "-c", src, "-o", out]))

    log = []
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        for (out, cmd, key), text in zip(tasks, ex.map(lambda t: _run(t[1], verbose), tasks)):
            stamp.mark(out, key)
            log.append((out.name, text))
    for name, text in log:
        if verbose and "registers" in text:
            lines = [l for l in text.splitlines() if "registers" in l or "spill" in l]
            print(f"[ptxas] {name}: " + " | ".join(l.strip() for l in lines[:12]))

    arts = {}
    # ---- link -----------------------------------------------------------------------------------
    def link(out: Path, objs, cmd):
        key = _sha(objs, " ".join(map(str, cmd)))
        if not stamp.fresh(out, key):
            _run(cmd, verbose)
            stamp.mark(out, key)
        arts[out.name] = str(out)

    ext = PKG / "_C.so"
    link(ext, cu_objs + host_objs + ext_objs,
         [CXX, "-shared", "-o", ext, *cu_objs, *host_objs, *ext_objs, *tlink])

    # ---- the same kernels, region layer and monitor as a plain C library (no Python, no PyTorch) -------------
    core = LIB / "libfuselink.so"
    link(core, cu_objs + host_objs,
         [CXX, "-shared", "-o", core, *cu_objs, *host_objs, f"-L{CUDA_HOME}/lib64", f"-Wl,-rpath,{CUDA_HOME}/lib64", "-lcudart",
          "-ldl", "-lrt", "-lpthread"])

    if net_objs:
        plug = LIB / "libnccl-net-fuselink.so"
        link(plug, net_objs + host_objs,
             [CXX, "-shared", "-Wl,-soname,libnccl-net-fuselink.so", "-o", plug, *net_objs, *host_objs, "-ldl", "-lrt", "-lpthread"])
        mon_src = CSRC / "monitor" / "monitor_main.cc"
        if mon_src.exists():
            mon = LIB / "fuselink-monitor"
            link(mon, [mon_src, host_objs[1]],
                 [CXX, *CXX_FLAGS, "-o", mon, mon_src, host_objs[1], "-lrt", "-lpthread"])
        har_src = CSRC / "net" / "harness_main.cc"
        if har_src.exists():
            har = LIB / "fl_net_harness"
            link(har, [har_src], [CXX, *CXX_FLAGS, "-o", har, har_src, "-ldl", "-lpthread"])

    stamp.save()
    return arts


def build_sanitized(kind: str = "address,undefined", verbose: bool = False) -> dict:
    """Sanitizer builds of the host-side code (plugin, harness, monitor stress driver) under ``lib/san-<kind>/``.

    ``kind`` is what goes after ``-fsanitize=``: "address,undefined" or "thread".  Used by the CPU test tier; the
    default build never links a sanitizer run time."""
    tag = kind.replace(",", "-")
    out = LIB / f"san-{tag}"
    out.mkdir(parents=True, exist_ok=True)
    flags = ["-O1", "-g", "-std=c++17", "-fPIC", f"-fsanitize={kind}", "-fno-omit-frame-pointer", "-pthread",
             f"-I{CUDA_HOME}/include"]
    net = [CSRC / "net" / f"{n}.cc" for n in NET_SRCS if (CSRC / "net" / f"{n}.cc").exists()]
    host = [CSRC / "mem" / "vmm.cc", CSRC / "monitor" / "monitor.cc"]
    plug, har, stress = out / "libnccl-net-fuselink.so", out / "fl_net_harness", out / "monitor_stress"
    stamp = _Stamp()
    hdrs = _headers()
    jobs = [
        (plug, net + host, [CXX, *flags, "-shared", "-o", plug, *net, *host, "-ldl", "-lrt", "-lpthread"]),
        (har, [CSRC / "net" / "harness_main.cc"], [CXX, *flags, "-o", har, CSRC / "net" / "harness_main.cc", "-ldl", "-lpthread"]),
        (stress, [CSRC / "monitor" / "monitor_stress.cc", host[1]],
         [CXX, *flags, "-o", stress, CSRC / "monitor" / "monitor_stress.cc", host[1], "-lrt", "-lpthread"]),
    ]
    todo = []
    for o, srcs, cmd in jobs:
        key = _sha(list(srcs) + hdrs, " ".join(map(str, cmd)))
        if not stamp.fresh(o, key):
            todo.append((o, cmd, key))
    def run_with_fallback(t):
        # the configured compiler may ship without the sanitizer run times: fall back to the system one
        cmd = t[1]
        last = None
        for cxx in dict.fromkeys([cmd[0], "/usr/bin/g++", "g++"]):
            try:
                return _run([cxx, *cmd[1:]], verbose)
            except RuntimeError as e:
                last = e
        raise last

    with ThreadPoolExecutor(max_workers=3) as ex:
        list(ex.map(run_with_fallback, todo))
    for o, _, key in todo:
        stamp.mark(o, key)
    stamp.save()
    return {"plugin": str(plug), "harness": str(har), "monitor_stress": str(stress)}


if __name__ == "__main__":
    out = build_all(verbose="-q" not in sys.argv)
    for k, v in out.items():
        print(f"built {k}: {v}")
