"""The C++ host runtime under include/qwen3: a host program written against the public headers alone builds with
a plain C++17 compiler and passes the cache's checks; the kernels' C header compiles as C and names every entry
point that the CUDA sources export; and the step metadata packed in C++ is what the layout says."""
import glob
import os
import re
import shutil
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE = os.path.join(ROOT, "qwen3-runtime-byyourself_b200")
INCLUDE = os.path.join(PACKAGE, "include")


def compiler(name):
    path = shutil.which(name)
    if path is None:
        pytest.skip(f"{name} is not installed")
    return path


def test_a_host_program_against_the_headers_alone(tmp_path):
    exe = str(tmp_path / "host_runtime_test")
    build = subprocess.run([compiler("g++"), "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", INCLUDE,
                            os.path.join(ROOT, "tests", "cpp", "host_runtime_test.cpp"), "-o", exe],
                           capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and run.stdout.strip().endswith("ok"), run.stdout[-2000:] + run.stderr[-2000:]


def test_the_kernels_header_is_c_and_names_every_exported_entry_point(tmp_path):
    source = tmp_path / "use.c"
    source.write_text('#include "qwen3/kernels.h"\nint main(void) { return q3_gemm_tcgen05_mid_splits(1, 1, 1) == -12345; }\n')
    check = subprocess.run([compiler("gcc"), "-std=c99", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-I", INCLUDE, str(source)],
                           capture_output=True, text=True, timeout=120)
    assert check.returncode == 0, check.stderr[-3000:]
    header = open(os.path.join(INCLUDE, "qwen3", "kernels.h")).read()
    declared = set(re.findall(r"\b(q3_\w+)\s*\(", header))
    exported = set()
    for path in glob.glob(os.path.join(PACKAGE, "csrc", "*.cu")):
        text = open(path).read()
        for name in re.findall(r"Q3_EXPORT\s+[\w\s\*]+?\b(q3_\w+)\s*\(", text):
            if "##" in name:
                continue
            exported.add(name)
        for name in re.findall(r"Q3_EXPORT\s+[\w\s\*]+?\b(q3_\w+)##SUFFIX", text):
            exported.update({name + "f32", name + "bf16"})
    exported.discard("q3_attention_decode_bf16_static")          # declared in its own header, beside its source
    assert exported and exported <= declared, sorted(exported - declared)


def test_step_metadata_packed_by_the_host_runtime():
    from qwen3_b200.cache import CacheBook, CacheNeed
    need = CacheNeed("full", 2, 16)
    book = CacheBook([need, CacheNeed("window", 1, 16, window=70)], max_tokens=6 * 64, max_seq_len=3 * 64, n_slots=3)
    a, b = book.alloc_slot(), book.alloc_slot()
    book.reserve([(a, 65), (b, 3)])
    book.commit([(a, 65), (b, 3)])
    book.reserve([(b, 2), (a, 1)])
    offsets, total = book.step_layout(3, 2, 2)
    assert offsets[0] == 0 and all(o % 4 == 0 for o in offsets) and len(offsets) == 7 + 2 and total % 4 == 0
    out = np.full(total, -7, dtype=np.int32)
    book.pack_step(np.array([b, a], dtype=np.int32), np.array([2, 1], dtype=np.int64), np.array([7, 8, 9], dtype=np.int32),
                   np.array([1, 2], dtype=np.int32), out)
    ids, seq, pos, slots, start, pos0, want = (out[o:] for o in offsets[:7])
    assert list(ids[:3]) == [7, 8, 9] and list(seq[:3]) == [0, 0, 1] and list(pos[:3]) == [3, 4, 65]
    assert list(slots[:2]) == [b, a] and list(start[:3]) == [0, 2, 3] and list(pos0[:2]) == [3, 65] and list(want[:2]) == [1, 2]
    P = book.pages_per_slot
    for g, o in enumerate(offsets[7:]):
        table = out[o:o + 2 * P].reshape(2, P)
        assert np.array_equal(table, book.page_rows(g, [b, a]))
    book.commit([(b, 2), (a, 1)])
    offsets, total = book.step_layout(4, 4, 4)
    out = np.full(total, -7, dtype=np.int32)
    book.pack_decode_step(4, np.array([a, b], dtype=np.int32), np.array([11, 12], dtype=np.int32), out)
    assert list(out[offsets[0]:offsets[0] + 4]) == [11, 12, 0, 0] and list(out[offsets[2]:offsets[2] + 4]) == [66, 5, 0, 0]
    assert list(out[offsets[3]:offsets[3] + 4]) == [a, b, book.n_slots, book.n_slots]
    table = out[offsets[7]:offsets[7] + 4 * P].reshape(4, P)
    assert np.array_equal(table[:2], book.page_rows(0, [a, b])) and (table[2:] == book.n_pages).all()
