"""Golden values for optimizer tests.

AdaScale gains for a ``Linear(2, 2)`` model whose loss is ``model(x).sum()``, two gradient passes per step
(accumulation or two ranks).  The values follow from the AdaScale estimator in closed form and match the ones
fairscale publishes in fairscale/fair_dev/testing/golden_testing_data.py:9-49.
"""

adascale_test_data = [
    {"input": [[1.0, 0], [0, 1.0]], "expected_gain": 4.0 / 3, "expected_grad": [[0.5, 0.5], [0.5, 0.5]], "expected_bias_grad": [1.0, 1.0]},
    {"input": [[1.0, 1.0], [1.0, 1.0]], "expected_gain": 1.0000001249999846, "expected_grad": [[1.0, 1.0], [1.0, 1.0]], "expected_bias_grad": [1.0, 1.0]},
    {"input": [[-1.0, 1.0], [1.0, -1.0]], "expected_gain": 2.0, "expected_grad": [[0.0, 0.0], [0.0, 0.0]], "expected_bias_grad": [1.0, 1.0]},
    {"input": [[1.0, 4.0], [5.0, 0.5]], "expected_gain": 1.4688796680497926, "expected_grad": [[3.0, 2.25], [3.0, 2.25]], "expected_bias_grad": [1.0, 1.0]},
    {"input": [[-0.2, 3.0], [5.0, 0.5]], "expected_gain": 1.8472893901708, "expected_grad": [[2.4000000953674316, 1.75], [2.4000000953674316, 1.75]], "expected_bias_grad": [1.0, 1.0]},
    # two steps: exercises the moving average
    {"inputs": [[[-0.2, 3.3], [5.2, 0.7]], [[1.0, 4.0], [3.1, 0.1]]], "expected_gain": 1.6720968158031417,
     "expected_grad": [[2.049999952316284, 2.049999952316284], [2.049999952316284, 2.049999952316284]], "expected_bias_grad": [1.0, 1.0]},
]

# Two ranks, ``Linear(3, 1, bias=False)`` with loss ``model(x).sum()``: the local gradient of a rank is its input, so the
# averaged gradient, the Pearson correlation of the two ranks' gradients and the cosine between consecutive averaged
# gradients follow by hand; same cases as fairscale/fair_dev/testing/golden_testing_data.py:51-63.
corr_mean_test_data = [
    {
        "inputs": [[[1.0, 0.0, 2.0], [2.0, 0.0, 1.0]], [[0.0, 1.0, 2.0], [2.0, 1.0, 0]], [[3.0, 1.0, 2.0], [2.0, 1.0, -1.0]]],
        "expected_grad": [[1.5, 0.0, 1.5], [1.0, 1.0, 1.0], [2.5, 1.0, 0.5]],
        "expected_corr": [0.5, -1.0, 0.327327],
        "expected_cos_similarity": [float("nan"), 0.8165, 0.8433],
    }
]
