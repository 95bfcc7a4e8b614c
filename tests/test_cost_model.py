"""The shipped cost-model file and its evaluator: schema the reference's lifecycle router
reads (ra_runtime_router.py:73-86), least-squares fit round trip, lifecycle ranking."""
import json
import math

import numpy as np

from ra_spmm_b200 import cost_model as CM


def test_design_row_terms():
    x = CM.design_rows(1000, 5000, 64, 5.0, 0.5)
    assert x.shape == (7,) and x[0] == 1.0
    assert math.isclose(x[1], math.log1p(1000)) and math.isclose(x[4], math.log1p(5000 * 64))
    assert math.isclose(x[5], math.log1p(5.0)) and math.isclose(x[6], math.log1p(0.5))
    assert CM.design_rows([10, 20], 100, 32, 1.0, 1.0).shape == (2, 7)


def test_shipped_model_schema_and_sanity():
    doc = json.loads(CM.SHIPPED_MODEL.read_text())
    model = CM.CostModel.load()
    assert set(CM.PORTFOLIO) <= set(model.kernels())
    for k in CM.PORTFOLIO:
        km = doc["kernels"][k]                      # the keys the reference's router indexes
        assert len(km["setup_coefficients"]) == 7 and len(km["warm_coefficients"]) == 7
        assert all(math.isfinite(c) for c in km["setup_coefficients"] + km["warm_coefficients"])
    # a plan-free kernel must not be predicted to cost more set-up than a tile plan build
    x = CM.design_rows(1 << 20, 11_000_000, 128, 10.8, 6.8)
    assert model.costs_ms("CSR_DIRECT", x)[0] <= model.costs_ms("TC_DIRECT", x)[0]


def test_fit_recovers_a_log_linear_law_and_ranks_by_lifecycle(tmp_path):
    rng = np.random.default_rng(0)
    true_setup = np.array([0.5, 0.1, 0.2, 0.0, 0.0, 0.05, 0.0])
    true_warm = np.array([-3.0, 0.0, 0.0, 0.0, 0.4, 0.0, 0.1])
    rows = []
    for _ in range(40):
        x = CM.design_rows(int(rng.integers(1e3, 1e6)), int(rng.integers(1e4, 1e8)),
                           int(rng.choice([32, 64, 128, 256])), float(rng.uniform(1, 300)),
                           float(rng.uniform(0, 8)))
        rows.append((x, float(np.exp(x @ true_setup)), float(np.exp(x @ true_warm))))
    m = CM.CostModel.fit({"A": rows})
    assert np.allclose(m.setup["A"], true_setup, atol=1e-6) and np.allclose(m.warm["A"], true_warm, atol=1e-6)
    m.save(tmp_path / "m.json")
    again = CM.CostModel.load(tmp_path / "m.json")
    assert np.allclose(again.warm["A"], m.warm["A"])
    # lifecycle: a cheap-to-build slow kernel wins one call, a costly fast one wins a thousand
    flat = lambda ms: [math.log(ms), 0, 0, 0, 0, 0, 0]
    two = CM.CostModel({"SLOW": {"setup_coefficients": flat(0.1), "warm_coefficients": flat(0.5)},
                        "FAST": {"setup_coefficients": flat(50.0), "warm_coefficients": flat(0.25)}})
    x = CM.design_rows(1000, 5000, 64, 5.0, 0.5)
    one, many = two.lifecycle_ms(x, 1), two.lifecycle_ms(x, 1000)
    assert min(one, key=one.get) == "SLOW" and min(many, key=many.get) == "FAST"
    assert two.lifecycle_ms(x, 1, allowed={"SLOW": False, "FAST": True}).keys() == {"FAST"}
