from .pool import Pool, CatBoostError, to_pool  # noqa: F401
