"""TEST INFRASTRUCTURE ONLY.  Recipe that compiles the reference's own host C++
for this path, from the sources where they lie, into ``oracle/_ref/``.

Two artefacts are produced (both git-ignored; they travel with the work tree):

``oracle/_ref/libhybrid_cpp.so``
    ``training/torch_rec_v1/hybrid_torchrec/src/{bind_torch_lib.cpp,ids_process/*.cpp}``
    unchanged: ``torch.classes.hybrid.IdsMapper``,
    ``torch.ops.hybrid.block_bucketize_sparse_features_cpu``.
``oracle/_ref/libref_embcache.so``
    ``torchrec_embcache/csrc/{embedding_cache/swap_manager.cpp,
    feature_filter/feature_filter.cpp, feature_filter/evict_feature_record.cpp,
    utils/logger.cpp}`` unchanged, plus ``oracle/ref_embcache_harness.cpp`` (a
    flat C ABI over ``SwapManager`` / ``FeatureFilter``).

``oracle/_ref/libref_manager.so``
    the whole ``EmbcacheManager`` (host store, ``Save`` / ``Load``) plus
    ``oracle/ref_manager_harness.cpp``; used to write and read checkpoints with the
    reference's own code.

No reference source is copied into this repository.  The reference tree is
found through ``RECSDK_REFERENCE_ROOT`` or, when that is unset, as a checkout
named ``reference`` beside this repository's own directory.  When neither
exists the recipe does nothing and whatever is already in ``oracle/_ref`` is
used as is.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def reference_root() -> str | None:
    root = os.environ.get("RECSDK_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return root if os.path.isdir(os.path.join(root, "training", "torch_rec_v1")) else None


def _torch_flags():
    import torch

    tdir = os.path.dirname(torch.__file__)
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    inc = [f"-I{tdir}/include", f"-I{tdir}/include/torch/csrc/api/include"]
    link = [f"-L{tdir}/lib", "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{tdir}/lib"]
    return abi, inc, link


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    print("[oracle/build_ref]", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build_hybrid(ref: str) -> str:
    src = os.path.join(ref, "training", "torch_rec_v1", "hybrid_torchrec", "src")
    sources = [os.path.join(src, "bind_torch_lib.cpp")] + sorted(glob.glob(os.path.join(src, "ids_process", "*.cpp")))
    out = os.path.join(OUT, "libhybrid_cpp.so")
    if _newer(out, sources):
        return out
    abi, inc, link = _torch_flags()
    _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fopenmp", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
          f"-I{src}", f"-I{src}/ids_process", *inc, *sources, "-o", out, *link])
    return out


def build_embcache(ref: str) -> str:
    src = os.path.join(ref, "training", "torch_rec_v1", "torchrec_embcache", "src", "torchrec_embcache", "csrc")
    sources = [
        os.path.join(src, "embedding_cache", "swap_manager.cpp"),
        os.path.join(src, "feature_filter", "feature_filter.cpp"),
        os.path.join(src, "feature_filter", "evict_feature_record.cpp"),
        os.path.join(src, "utils", "logger.cpp"),
        os.path.join(HERE, "ref_embcache_harness.cpp"),
    ]
    out = os.path.join(OUT, "libref_embcache.so")
    if _newer(out, sources):
        return out
    abi, inc, link = _torch_flags()
    _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fopenmp", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
          f"-I{src}", *inc, *sources, "-o", out, *link])
    return out


def build_manager(ref: str) -> str:
    """The reference's whole EmbcacheManager (host store, Save / Load) behind oracle/ref_manager_harness.cpp.  Its
    sources include a bounds-checked C library header that is not in the tree: oracle/ref_shims/securec.h stands in
    (memcpy_s / memset_s only)."""
    src = os.path.join(ref, "training", "torch_rec_v1", "torchrec_embcache", "src", "torchrec_embcache", "csrc")
    sources = [os.path.join(src, *p) for p in (
        ("embedding_cache", "embcache_manager.cpp"), ("embedding_cache", "swap_manager.cpp"),
        ("feature_filter", "feature_filter.cpp"), ("feature_filter", "evict_feature_record.cpp"),
        ("utils", "logger.cpp"), ("file_system", "file_system_handler.cpp"),
        ("file_system", "local_file_system", "local_file_system.cpp"), ("emb_table", "emb_mem_pool.cpp"),
        ("hash_table", "fast_hashmap.cpp"), ("hash_table", "hash_bucket.cpp"))]
    sources.append(os.path.join(HERE, "ref_manager_harness.cpp"))
    out = os.path.join(OUT, "libref_manager.so")
    if _newer(out, sources):
        return out
    import sysconfig

    abi, inc, link = _torch_flags()
    # the manager's headers pull in torch's Python-facing headers (it is the body of a pybind module)
    py_inc = sysconfig.get_paths()["include"]
    _run(["g++", "-O1", "-std=c++17", "-fPIC", "-shared", "-fopenmp", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
          f"-I{src}", f"-I{os.path.join(HERE, 'ref_shims')}", f"-I{py_inc}", *inc, *sources, "-o", out, *link])
    return out


def build_all(verbose: bool = True) -> bool:
    """Build both artefacts if the reference tree is present.  Returns True when
    the reference tree was found (built or already current)."""
    ref = reference_root()
    if ref is None:
        if verbose:
            print("[oracle/build_ref] reference tree not present; using prebuilt oracle/_ref as is")
        return False
    os.makedirs(OUT, exist_ok=True)
    build_hybrid(ref)
    build_embcache(ref)
    try:
        build_manager(ref)
    except subprocess.CalledProcessError:  # optional third artefact: the tests that need it skip without it
        if verbose:
            print("[oracle/build_ref] the reference manager did not build; checkpoint cross-checks will skip")
    return True


if __name__ == "__main__":
    sys.exit(0 if build_all() or True else 1)
