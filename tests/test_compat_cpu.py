"""The source-level stand-in for the reference's slime/core/pseudopod.cu (include/compat/pseudopod.cu): it
compiles on its own, the reference's translation unit compiles unchanged against it (when a checkout of the
reference sits beside this repository), and the oracle's reading of the reference's weight bundle is what plain
slicing gives."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from oracle import ca_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
REFERENCE = os.environ.get("SLIME_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-rdc=true", "--expt-relaxed-constexpr", "-w"]


def _env():
    env = dict(os.environ)
    env.pop("CC", None); env.pop("CXX", None)
    return env


@pytest.mark.skipif(not os.path.exists(NVCC), reason="needs nvcc")
def test_compat_file_compiles_alone(tmp_path):
    src = tmp_path / "tu.cu"
    src.write_text('#include "compat/pseudopod.cu"\nint main() { return 0; }\n')
    subprocess.run([NVCC, *FLAGS, "-I" + os.path.join(ROOT, "include"), "-c", str(src), "-o", str(tmp_path / "tu.o")],
                   check=True, env=_env())


@pytest.mark.skipif(not os.path.exists(NVCC) or not os.path.exists(os.path.join(REFERENCE, "slime", "core", "organism.cu")),
                    reason="needs nvcc and a checkout of the reference beside this repository")
def test_reference_translation_unit_compiles_against_compat(tmp_path):
    """main.cu -> runtime.cu -> organism.cu, all unchanged, with only core/pseudopod.cu swapped (in a scratch copy)."""
    shutil.copy(os.path.join(REFERENCE, "main.cu"), tmp_path / "main.cu")
    shutil.copytree(os.path.join(REFERENCE, "slime"), tmp_path / "slime")
    shutil.copy(os.path.join(ROOT, "include", "compat", "pseudopod.cu"), tmp_path / "slime" / "core" / "pseudopod.cu")
    subprocess.run([NVCC, *FLAGS, "-I" + str(tmp_path), "-I" + os.path.join(ROOT, "include"), "-c",
                    str(tmp_path / "main.cu"), "-o", str(tmp_path / "main.o")], check=True, env=_env())
    assert os.path.getsize(tmp_path / "main.o") > 0


def test_oracle_weights_from_reference_layout():
    rng = np.random.default_rng(3)
    per = rng.standard_normal((8, 512, 256)).astype(np.float32)
    inter = rng.standard_normal((8, 512, 256)).astype(np.float32)
    val = rng.standard_normal((8, 256, 512)).astype(np.float32)
    mix = (np.eye(8) + 0.01 * rng.standard_normal((8, 8))).astype(np.float32)
    flow = rng.random((8, 9)).astype(np.float32)
    Wp, Wi, Wv, Wo, K = ca_oracle.weights_from_reference_layout(per, inter, val, mix, flow)
    assert np.array_equal(Wp, per[:, :64, :64]) and np.array_equal(Wi, inter[:, :64, :64])
    folded = ((val[:, 0:64, :64] + val[:, 64:128, :64]) + val[:, 128:192, :64]) + val[:, 192:256, :64]
    assert np.array_equal(Wv, folded)
    assert np.array_equal(K, flow)
    Wo4 = Wo.reshape(8, 64, 64)
    for h in range(8):
        assert np.allclose(Wo4[h], np.eye(64) * mix[:, h].astype(np.float64).mean(), atol=1e-7)


def test_oracle_field_from_state():
    rng = np.random.default_rng(4)
    X = rng.random((2, 5, 7, 64)).astype(np.float32)
    assert np.allclose(ca_oracle.field_from_state(X), X.astype(np.float64).mean(-1), atol=1e-7)


def test_output_projection_folds_the_reference_head_mixing():
    """tests/golden/ref_mix_heads.json holds what the reference's own mix_heads_kernel wrote on a B200 for six cells
    (oracle/ref_mix_harness.cu, `make -C oracle ref_mix`).  The contract state has 64 channels where the reference's
    mixed output has 8 x 64; slime_ca_set_weights_reference_layout folds the 8 x 8 mixing followed by the mean of the
    eight output heads into Wo.  Applied to the same head outputs that Wo must give the mean of the reference
    kernel's output heads."""
    import json
    ref = json.load(open(os.path.join(ROOT, "tests", "golden", "ref_mix_heads.json")))
    f = lambda a: np.array(a, dtype=np.uint32).view(np.float32)
    mix = f(ref["mixing"]).reshape(8, 8)
    z = np.zeros((8, 512, 256), np.float32)
    Wo = ca_oracle.weights_from_reference_layout(z, z, np.zeros((8, 256, 512), np.float32), mix, np.zeros((8, 9), np.float32))[3]
    assert len(ref["cells"]) == 6
    for cell in ref["cells"]:
        v = f(cell["head_outputs"]).astype(np.float64)                   # [8 heads * 64]
        out = f(cell["final_output"]).astype(np.float64).reshape(8, 64)  # [out_head][c]
        # the reference kernel itself: out[o][c] = sum_in mixing[o][in] * v[in][c]
        assert np.abs(out - mix.astype(np.float64) @ v.reshape(8, 64)).max() < 1e-6
        assert np.abs(v @ Wo.astype(np.float64) - out.mean(axis=0)).max() < 1e-6


def test_genome_hash_matches_the_reference_kernel():
    """tests/golden/ref_elite.json holds what the reference's own create_elite_kernel (slime/memory/archive.cu:66-82,
    run on a B200 by oracle/ref_elite_harness.cu) wrote for four seeded genomes; the restated hash reproduces every
    genome_hash, and the record keeps fitness, coherence, effective rank and generation as given."""
    import json
    import struct
    from oracle import ca_oracle
    z = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_elite.json")))
    assert len(z["cases"]) == 4
    for i, c in enumerate(z["cases"]):
        genome = np.array(c["genome"], dtype=np.uint32).view(np.float32)
        assert ca_oracle.genome_hash(genome) == int(c["genome_hash"])
        as_f = lambda u: struct.unpack("<f", struct.pack("<I", u))[0]
        assert as_f(c["fitness"]) == 1.5 + i and as_f(c["coherence"]) == 0.25 * i and as_f(c["effective_rank"]) == 6.0 - i
        assert c["generation"] == 40 + 1000 * i
    assert any(u >= 0x80000000 for c in z["cases"] for u in c["genome"])      # negative values: the 32-bit sum wraps
