"""Golden values for optimizer tests.

AdaScale gains for a ``Linear(2, 2)`` model whose loss is ``model(x).sum()``, two gradient passes per step
(accumulation or two ranks).  The values follow from the AdaScale estimator in closed form and match the ones
fairscale publishes in fairscale/fair_dev/testing/golden_testing_data.py:9-49.
"""

_NAN = float("nan")
_ONES = [1.0, 1.0]  # the bias gradient of ``model(x).sum()`` is one per output, whatever the input


def _square(row):
    """Both output rows of the weight see the same gradient."""
    return [list(row), list(row)]


# (the two inputs of one step, gain after the step, one row of the averaged weight gradient)
_ONE_STEP = [
    ([[1.0, 0], [0, 1.0]], 4.0 / 3, [0.5, 0.5]),
    ([[1.0, 1.0], [1.0, 1.0]], 1.0000001249999846, [1.0, 1.0]),
    ([[-1.0, 1.0], [1.0, -1.0]], 2.0, [0.0, 0.0]),
    ([[1.0, 4.0], [5.0, 0.5]], 1.4688796680497926, [3.0, 2.25]),
    ([[-0.2, 3.0], [5.0, 0.5]], 1.8472893901708, [2.4000000953674316, 1.75]),
]
# two steps: exercises the moving average
_TWO_STEPS = ([[[-0.2, 3.3], [5.2, 0.7]], [[1.0, 4.0], [3.1, 0.1]]], 1.6720968158031417, [2.049999952316284, 2.049999952316284])

adascale_test_data = [
    {"input": x, "expected_gain": gain, "expected_grad": _square(row), "expected_bias_grad": list(_ONES)} for x, gain, row in _ONE_STEP
] + [
    {"inputs": _TWO_STEPS[0], "expected_gain": _TWO_STEPS[1], "expected_grad": _square(_TWO_STEPS[2]), "expected_bias_grad": list(_ONES)}
]

# Two ranks, ``Linear(3, 1, bias=False)`` with loss ``model(x).sum()``: the local gradient of a rank is its input, so the
# averaged gradient, the Pearson correlation of the two ranks' gradients and the cosine between consecutive averaged
# gradients follow by hand; same cases as fairscale/fair_dev/testing/golden_testing_data.py:51-63.
_RANK_INPUTS = [[[1.0, 0.0, 2.0], [2.0, 0.0, 1.0]], [[0.0, 1.0, 2.0], [2.0, 1.0, 0]], [[3.0, 1.0, 2.0], [2.0, 1.0, -1.0]]]
corr_mean_test_data = [
    {
        "inputs": _RANK_INPUTS,
        "expected_grad": [[(a + b) / 2 for a, b in zip(*pair)] for pair in _RANK_INPUTS],
        "expected_corr": [0.5, -1.0, 0.327327],
        "expected_cos_similarity": [_NAN, 0.8165, 0.8433],
    }
]
