"""Sampling from the Gaussian-process posterior that gradient boosting converges to (Kernel Gradient Boosting, algorithm 4
of "Gradient Boosting Performs Gaussian Process Inference", Ustimenko, Beliakov, Prokhorenkova;
catboost/python-package/catboost/core.py ``sample_gaussian_process``).

One sample = prior function + posterior correction:
  1. the prior is an ensemble of ``prior_iterations`` random trees: structures drawn by training on pure noise with a
     vanishing learning rate and an overwhelming score noise (so every split is random), leaf values drawn as independent
     normals with deviation sqrt(N / sqrt(leaf weight)), the whole ensemble scaled by sigma / sqrt(prior_iterations);
  2. the posterior model is trained on ``y - prior(X) + N(0, delta^2)`` with RMSE, score noise ``random_strength`` and the
     model shrinkage (random_strength / sigma)^2 / N that makes the boosting iterations a Langevin-type sampler;
  3. the sample is the sum of the two models.
"""
from __future__ import annotations

import numpy as np


def sample_gaussian_process(X, y, eval_set=None, cat_features=None, text_features=None, embedding_features=None,
                            random_seed=None, samples=10, posterior_iterations=900, prior_iterations=100,
                            learning_rate=0.1, depth=6, sigma=0.1, delta=0, random_strength=0.1,
                            random_score_type="Gumbel", eps=1e-4, verbose=False):
    """Returns ``samples`` CatBoostRegressor models, each one draw from the posterior GP with prior
    f ~ GP(0, sigma^2 K + delta^2 I)."""
    from .core import CatBoostRegressor, sum_models
    if not (sigma > 0 and samples > 0 and random_strength > 0 and eps > 0):
        raise ValueError("sigma, samples, random_strength and eps must be positive")
    rng = np.random.default_rng(0 if random_seed is None else random_seed)
    seeds = rng.integers(0, 2 ** 31 - 1, size=(samples, 2))
    y = np.asarray(y, dtype=np.float64).reshape(-1)
    N = len(y)
    shrink = (random_strength / sigma) ** 2 / N
    fit_kw = dict(cat_features=cat_features, text_features=text_features, embedding_features=embedding_features)
    fit_kw = {k: v for k, v in fit_kw.items() if v is not None}
    common = dict(loss_function="RMSE", bootstrap_type="No", depth=depth, boost_from_average=False, score_function="L2",
                  boosting_type="Plain", random_score_type=random_score_type, allow_writing_files=False)
    out = []
    for k in range(samples):
        prior = CatBoostRegressor(random_seed=int(seeds[k, 0]), iterations=prior_iterations, learning_rate=eps,
                                  random_strength=1.0 / eps, l2_leaf_reg=0, verbose=False, **common)
        prior.fit(X, rng.normal(scale=eps, size=N), use_best_model=False, **fit_kw)
        values = []
        for t in prior._model.trees:
            w = np.maximum(np.asarray(t.leaf_weights, dtype=np.float64).reshape(-1), 1.0)
            values.append(rng.normal(size=len(w)) * np.sqrt(N / np.sqrt(w)))
        prior.set_leaf_values(np.concatenate(values))
        scale, bias = prior.get_scale_and_bias()
        k_scale = sigma / np.sqrt(prior_iterations)
        prior.set_scale_and_bias(scale * k_scale, np.asarray(bias, dtype=np.float64) * k_scale)
        target = y - np.asarray(prior.predict(X), dtype=np.float64) + rng.normal(scale=delta, size=N)
        post = CatBoostRegressor(random_seed=int(seeds[k, 1]), iterations=posterior_iterations, learning_rate=learning_rate,
                                 model_shrink_rate=shrink, random_strength=random_strength, l2_leaf_reg=0, verbose=verbose,
                                 **common)
        post.fit(X, target, eval_set=eval_set, use_best_model=False, **fit_kw)
        out.append(sum_models([prior, post]))
    return out
