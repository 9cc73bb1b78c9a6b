"""Trainers (boosting loop, device engine, general learner, objectives, CTRs).

``catboost_b200.train`` is also the name of the functional entry point ``train(pool, params, ...)`` exported by the top
level package; importing this sub-package rebinds that attribute to the module, so the module itself is made callable
and forwards to the function: ``catboost_b200.train(...)`` works whichever object the name holds.
"""
import sys
import types


class _CallableTrainModule(types.ModuleType):
    def __call__(self, *args, **kwargs):
        from ..core import train as _train
        return _train(*args, **kwargs)


sys.modules[__name__].__class__ = _CallableTrainModule
