"""The native dataset-index builders under AddressSanitizer + UBSan (host code): edge shapes, no reports."""
import os
import subprocess
import sys

import pytest

from common import ROOT

CHILD = r"""
import os, sys, numpy as np
sys.path.insert(0, sys.argv[1])
os.environ["NEOX_DATA_LIB"] = sys.argv[2]
from gpt_neox_b200.data import helpers
rng = np.random.default_rng(0)
for n_docs, seq, epochs in [(1, 4, 1), (3, 1, 2), (200, 33, 3), (50, 2048, 1)]:
    sizes = rng.integers(1, 70, size=n_docs).astype(np.int32)
    doc_idx = np.concatenate([rng.permutation(n_docs) for _ in range(epochs)]).astype(np.int32)
    tpe = int(sizes.sum())
    if (epochs * tpe - 1) // seq < 1:
        continue
    a = helpers.build_sample_idx_int32(sizes, doc_idx, seq, epochs, tpe)
    b = helpers.build_sample_idx_numpy(sizes, doc_idx, seq, epochs, tpe)
    assert np.array_equal(a, b)
for w, size in [([1.0], 5), ([0.2, 0.8], 1), ([0.3, 0.3, 0.4], 1000)]:
    di = np.zeros(size, dtype=np.uint8); dsi = np.zeros(size, dtype=np.int64)
    helpers.build_blending_indices(di, dsi, np.array(w), len(w), size, False)
    assert di.max() < len(w)
print("SANITIZED-OK")
"""


def test_data_helpers_under_asan_ubsan(tmp_path):
    from gpt_neox_b200.build import build_data_helpers_sanitized
    gxx = asan = None
    for cand in (os.environ.get("CXX"), "/usr/bin/g++", "g++"):       # a compiler that ships the ASan runtime
        if not cand:
            continue
        try:
            path = subprocess.run([cand, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
        except OSError:
            continue
        if os.path.isabs(path) and os.path.exists(path):
            gxx, asan = cand, path
            break
    if gxx is None:
        pytest.skip("no compiler with an ASan runtime on this machine")
    lib = build_data_helpers_sanitized(tmp_path, cxx=gxx)
    env = dict(os.environ, LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:abort_on_error=1",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([sys.executable, "-c", CHILD, ROOT, str(lib)], capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0 and "SANITIZED-OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-4000:]
