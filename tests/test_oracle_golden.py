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
