"""CPU: the evaluate_inversed oracle (oracle/cpu/eval_inversed.c) against the golden vectors produced by the
reference's own Python, and against the closed-form known answer of the reference's test."""
import math

import numpy as np

from conftest import rel_inf
from oracle import cpu_oracle


def _cases(golden):
    return sorted({k.rsplit("_mixture", 1)[0] for k in golden if k.endswith("_mixture") and "grad" not in k})


def test_known_answer():
    # src/gmc/test_cpp_eval.py:25-28: one Gaussian, weight 1, S = 2 I, evaluated at its centre
    mixture = np.array([1.0, 0.0, 0.0, 2.0, 0.0, 0.0, 2.0], dtype=np.float64).reshape(1, 1, 1, 7)
    xes = np.zeros((1, 1, 1, 2))
    out = cpu_oracle.eval_forward(mixture, xes)
    assert abs(out[0, 0, 0] - math.sqrt(4.0) / (2 * math.pi)) < 1e-15


def test_oracle_f64_matches_reference_python(golden_eval):
    cases = _cases(golden_eval)
    assert len(cases) == 11
    for c in cases:
        m = golden_eval[c + "_mixture"].astype(np.float64)
        x = golden_eval[c + "_xes"].astype(np.float64)
        g = golden_eval[c + "_grad_out"].astype(np.float64)
        out = cpu_oracle.eval_forward(m, x)
        gm, gx = cpu_oracle.eval_backward(g, m, x)
        assert rel_inf(out, golden_eval[c + "_out"]) < 1e-12, c
        assert rel_inf(gm, golden_eval[c + "_grad_mixture"]) < 1e-11, c
        assert rel_inf(gx, golden_eval[c + "_grad_xes"]) < 1e-11, c


def test_oracle_f32_within_tolerance(golden_eval):
    # the fp32 instantiation is the timed CPU baseline; it must itself be inside the 1e-4 band
    for c in _cases(golden_eval):
        m = golden_eval[c + "_mixture"]
        x = golden_eval[c + "_xes"]
        g = golden_eval[c + "_grad_out"]
        out = cpu_oracle.eval_forward(m, x)
        gm, gx = cpu_oracle.eval_backward(g, m, x)
        assert rel_inf(out, golden_eval[c + "_out"]) < 1e-4, c
        assert rel_inf(out, golden_eval[c + "_out_f32ref"]) < 1e-4, c
        assert rel_inf(gm, golden_eval[c + "_grad_mixture"]) < 1e-4, c
        assert rel_inf(gx, golden_eval[c + "_grad_xes"]) < 1e-4, c
