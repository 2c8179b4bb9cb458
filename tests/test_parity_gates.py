"""pytest drives the parity gates (``parity/*_test.py``, standalone scripts in the reference's manner), each
in a subprocess of its own; a gate passes when it exits 0 and proves its work with ``PARITY-CHECKS: n``."""

import pytest

from parity import _gates

GATES = _gates.discover()


def test_the_gates_are_found():
    assert {"minimax_m3_config_test", "minimax_m3_cuttings_test", "minimax_m3_generate_test"} <= set(GATES)


@pytest.mark.parametrize("name", [n for n, gpu in GATES.items() if not gpu])
def test_gate_without_a_gpu(name):
    r = _gates.run_gate(name)
    assert r.ok and r.checks > 0, (r.why, r.output[-2000:])


@pytest.mark.gpu
@pytest.mark.parametrize("name", [n for n, gpu in GATES.items() if gpu])
def test_gate_on_the_gpu(name):
    r = _gates.run_gate(name)
    assert r.ok and r.checks > 0, (r.why, r.output[-2000:])


def test_a_gate_that_proves_no_work_fails(tmp_path, monkeypatch):
    """Exit code 0 is not enough: without a positive PARITY-CHECKS line the runner reports a failure."""
    fake = _gates.PARITY_DIR / "zz_vacuous_gate_for_the_runner_test.py"
    fake.write_text("print('nothing checked')\n")
    try:
        r = _gates.run_gate(fake.stem)
        assert not r.ok and "PARITY-CHECKS" in r.why
    finally:
        fake.unlink()
