"""Compiles csrc/*.cu into libtsm_b200.so for sm_100a with nvcc (in-tree, no JIT cache)."""
import glob
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBRARY = os.path.join(HERE, "libtsm_b200.so")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--threads", "0"]


EXTRA = {}  # per-file compiler flags


def nvcc():
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc was not found; the library cannot be built")
    return found


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def stale():
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return any(os.path.getmtime(p) > built for p in deps)


def build(verbose=False, force=False):
    """Builds the shared library when a source is newer than it; returns its path.  Several processes may ask at once (one per
    GPU under torch.distributed.run): a lock file lets one of them build while the others wait and then find it fresh."""
    import fcntl
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    with open(os.path.join(HERE, "build", ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _build_locked(verbose, force)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(verbose, force):
    if not force and not stale():
        return LIBRARY
    objects = []
    out_dir = os.path.join(HERE, "build")
    os.makedirs(out_dir, exist_ok=True)
    procs = []
    for src in sources():
        obj = os.path.join(out_dir, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(
                [os.path.getmtime(src)] + [os.path.getmtime(h) for h in glob.glob(os.path.join(CSRC, "*.cuh"))] +
                [os.path.getmtime(h) for h in glob.glob(os.path.join(HERE, "..", "include", "*.h"))]):
            continue
        cmd = [nvcc()] + FLAGS + EXTRA.get(os.path.basename(src), []) + ["-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + out)
        if verbose and out.strip():
            print(out)
    cmd = [nvcc(), "-shared", "-o", LIBRARY] + objects + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart_static", "-ldl",
                                                         "-lpthread", "-lrt"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return LIBRARY


if __name__ == "__main__":
    build(verbose=True)
