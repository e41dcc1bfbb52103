"""Pins the CPU restatement (oracle/) against the reference: for every golden fixture the oracle
must reproduce (a) what the reference's own emitted CPU code computed for the same inputs and
(b) the expected vectors checked into the reference's test-suite."""
from pathlib import Path

import numpy as np
import pytest

import graph_runner as gr

GOLDEN = sorted(p.stem for p in (Path(__file__).parent / "golden").glob("*.npz"))


def close(got, want, rel=1e-5):
    """|got - want| <= rel * max(|want|, rms(want)): the fp32 bound with a per-tensor floor."""
    floor = float(np.sqrt(np.mean(np.square(want)))) if want.size else 0.0
    return np.all(np.abs(got - want) <= rel * np.maximum(np.abs(want), floor) + 1e-30)


@pytest.fixture(scope="module")
def backend(oracle_lib):
    return gr.OracleBackend()


def test_fixture_inventory():
    assert len(GOLDEN) >= 30 and "MLP_C1" in GOLDEN and "ConvWithPadding" in GOLDEN


@pytest.mark.parametrize("name", GOLDEN)
def test_oracle_matches_reference_code(name, backend):
    fx = gr.load_fixture(name)
    for tag in ("A", "B"):
        if f"out{tag}" not in fx:
            continue
        ins = [fx[k] for k in sorted(fx) if k.startswith(f"in{tag}")]
        got = gr.run_graph(fx, ins, backend)
        want = fx[f"out{tag}"]
        assert got.shape == want.shape
        assert close(got, want), f"{name}/{tag}: max abs diff {np.abs(got - want).max():.3g}"


@pytest.mark.parametrize("name", [n for n in GOLDEN if "expected" in np.load(Path(__file__).parent / "golden" / f"{n}.npz").files])
def test_oracle_matches_checked_in_vectors(name, backend):
    fx = gr.load_fixture(name)
    ins = [fx[k] for k in sorted(fx) if k.startswith("inA")]
    got = gr.run_graph(fx, ins, backend)
    # the checked-in vectors carry 4-6 significant digits; the reference compares at 1e-3 absolute
    # (tests/alpaka/TestAlpakaCommon.h:10); 2e-4 is what their printed precision allows
    assert np.abs(got - fx["expected"]).max() <= 2e-4


# ---- the model configurations, pinned to the reference's emitted code at reduced size ---------------------------------
CONFIGS = Path(__file__).parent / "golden" / "configs"


def test_convnet_restatement_matches_reference_code(oracle_lib):
    """8 x (Conv3x3 -> BatchNormalization + Relu), GlobalAveragePool, Gemm on 2 images of 32 x 32: the reference ran Conv and
    BatchNormalization as separate operators; the restatement folds the normalisation into the convolution's epilogue."""
    import model_oracles as mo
    from oracle_api import Oracle
    from sofie_b200 import convnet
    fx = np.load(CONFIGS / "ConvNet_C4r.npz")
    got = mo.convnet_oracle(Oracle(oracle_lib), fx["x"], convnet.make_weights(int(fx["seed"]), False), False)
    assert close(got, fx["y"]), np.abs(got - fx["y"]).max()


def test_encoder_restatement_matches_reference_code(oracle_lib):
    """2 encoder layers, 2 sequences: the reference ran fp32 on the dequantised weights; the restatement keeps bf16 tensors
    and int8 weights with the scale in the epilogue.  Bar of the low-precision path: 2e-2 relative + 1e-2 absolute."""
    import model_oracles as mo
    from oracle_api import Oracle, bf16_bits_to_f32
    from sofie_b200 import encoder
    fx = np.load(CONFIGS / "Encoder_C5r.npz")
    w = encoder.make_weights(int(fx["seed"]), int(fx["layers"]), 512, 2048)
    got = bf16_bits_to_f32(mo.encoder_oracle(Oracle(oracle_lib), encoder.f32_to_bf16_bits(fx["x"]), w, int(fx["batch"]), 128, 512, 8))
    assert np.all(np.abs(got - fx["y"]) <= 2e-2 * np.abs(fx["y"]) + 1e-2), np.abs(got - fx["y"]).max()
