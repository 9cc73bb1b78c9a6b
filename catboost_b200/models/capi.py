"""ctypes view of the stand-alone evaluator library (``ops/cpu/cb_model_capi.h``).

The library is what programs in other languages link against (the interface of the reference's
catboost/libs/model_interface/c_api.h); this wrapper exists so that the Python tests can drive exactly that interface
and so that a Python service can apply a model without importing torch.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

_lib = None

_PREDICTION_TYPES = {"RawFormulaVal": 0, "Exponent": 1, "RMSEWithUncertainty": 2, "Probability": 3, "Class": 4,
                     "MultiProbability": 5}


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        from ..ops import native
        lib = ctypes.CDLL(str(native.build_model_lib()))
        vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        lib.ModelCalcerCreate.restype = vp
        lib.ModelCalcerDelete.argtypes = [vp]
        lib.ModelCalcerDelete.restype = None
        lib.GetErrorString.restype = ctypes.c_char_p
        for name, args in {
            "LoadFullModelFromFile": [vp, ctypes.c_char_p],
            "LoadFullModelFromBuffer": [vp, vp, sz],
            "SetPredictionType": [vp, ci],
            "SetPredictionTypeString": [vp, ctypes.c_char_p],
            "CalcModelPredictionFlat": [vp, sz, vp, sz, vp, sz],
            "CalcModelPredictionFlatStaged": [vp, sz, sz, sz, vp, sz, vp, sz],
            "CalcModelPredictionFlatTransposed": [vp, sz, vp, sz, vp, sz],
            "CalcModelPrediction": [vp, sz, vp, sz, vp, sz, vp, sz],
            "CalcModelPredictionSingle": [vp, vp, sz, vp, sz, vp, sz],
            "CalcModelPredictionWithHashedCatFeatures": [vp, sz, vp, sz, vp, sz, vp, sz],
            "PredictSpecificClassFlat": [vp, sz, vp, sz, ci, vp, sz],
            "EnableGPUEvaluation": [vp, ci],
            "CheckModelMetadataHasKey": [vp, ctypes.c_char_p, sz],
            "GetModelUsedFeaturesNames": [vp, vp, vp],
            "GetFloatFeatureIndices": [vp, vp, vp],
            "GetCatFeatureIndices": [vp, vp, vp],
        }.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = ctypes.c_bool
        for name in ("GetFloatFeaturesCount", "GetCatFeaturesCount", "GetTreeCount", "GetDimensionsCount",
                     "GetPredictionDimensionsCount"):
            fn = getattr(lib, name)
            fn.argtypes = [vp]
            fn.restype = sz
        lib.GetModelInfoValueSize.argtypes = [vp, ctypes.c_char_p, sz]
        lib.GetModelInfoValueSize.restype = sz
        lib.GetModelInfoValue.argtypes = [vp, ctypes.c_char_p, sz]
        lib.GetModelInfoValue.restype = vp
        lib.GetStringCatFeatureHash.argtypes = [ctypes.c_char_p, sz]
        lib.GetStringCatFeatureHash.restype = ci
        lib.GetIntegerCatFeatureHash.argtypes = [ctypes.c_longlong]
        lib.GetIntegerCatFeatureHash.restype = ci
        _lib = lib
    return _lib


class NativeModelError(RuntimeError):
    pass


def _row_pointers(a: np.ndarray):
    ptrs = (ctypes.c_void_p * a.shape[0])()
    base, stride = a.ctypes.data, a.strides[0]
    for i in range(a.shape[0]):
        ptrs[i] = base + i * stride
    return ptrs


class NativeModelCalcer:
    """A model handle of the stand-alone evaluator."""

    def __init__(self, path: Optional[str] = None, blob: Optional[bytes] = None):
        self._lib = library()
        self._h = self._lib.ModelCalcerCreate()
        if not self._h:
            raise NativeModelError("cannot create a model handle")
        if path is not None:
            self._check(self._lib.LoadFullModelFromFile(self._h, str(path).encode("utf-8")))
        elif blob is not None:
            buf = ctypes.create_string_buffer(blob, len(blob))
            self._check(self._lib.LoadFullModelFromBuffer(self._h, ctypes.cast(buf, ctypes.c_void_p), len(blob)))

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ModelCalcerDelete(h)

    def _check(self, ok):
        if not ok:
            raise NativeModelError((self._lib.GetErrorString() or b"").decode("utf-8", "replace"))

    # ---- description -------------------------------------------------------------------------------------------
    @property
    def tree_count(self) -> int:
        return int(self._lib.GetTreeCount(self._h))

    @property
    def dimensions(self) -> int:
        return int(self._lib.GetDimensionsCount(self._h))

    @property
    def prediction_dimensions(self) -> int:
        return int(self._lib.GetPredictionDimensionsCount(self._h))

    @property
    def float_features_count(self) -> int:
        return int(self._lib.GetFloatFeaturesCount(self._h))

    @property
    def cat_features_count(self) -> int:
        return int(self._lib.GetCatFeaturesCount(self._h))

    def _indices(self, fn):
        arr, cnt = ctypes.POINTER(ctypes.c_size_t)(), ctypes.c_size_t()
        self._check(fn(self._h, ctypes.byref(arr), ctypes.byref(cnt)))
        out = [int(arr[i]) for i in range(cnt.value)]
        ctypes.CDLL(None).free(arr)
        return out

    def float_feature_indices(self):
        return self._indices(self._lib.GetFloatFeatureIndices)

    def cat_feature_indices(self):
        return self._indices(self._lib.GetCatFeatureIndices)

    def used_feature_names(self):
        arr, cnt = ctypes.POINTER(ctypes.c_char_p)(), ctypes.c_size_t()
        self._check(self._lib.GetModelUsedFeaturesNames(self._h, ctypes.byref(arr), ctypes.byref(cnt)))
        raw = ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p))
        out = [ctypes.string_at(raw[i]).decode("utf-8") for i in range(cnt.value)]
        libc = ctypes.CDLL(None)
        libc.free.argtypes = [ctypes.c_void_p]
        for i in range(cnt.value):
            libc.free(raw[i])
        libc.free(ctypes.cast(arr, ctypes.c_void_p))
        return out

    def metadata(self, key: str) -> Optional[str]:
        k = key.encode("utf-8")
        if not self._lib.CheckModelMetadataHasKey(self._h, k, len(k)):
            return None
        n = self._lib.GetModelInfoValueSize(self._h, k, len(k))
        p = self._lib.GetModelInfoValue(self._h, k, len(k))
        return ctypes.string_at(p, n).decode("utf-8")

    def set_prediction_type(self, prediction_type: str):
        self._check(self._lib.SetPredictionTypeString(self._h, prediction_type.encode("ascii")))

    # ---- evaluation --------------------------------------------------------------------------------------------
    def _result(self, n):
        return np.empty((n, self.prediction_dimensions), dtype=np.float64)

    def predict_flat(self, X, tree_start: int = 0, tree_end: Optional[int] = None, transposed: bool = False) -> np.ndarray:
        """``X``: float32 [docs][flat features] (categorical columns hold the bits of the int hash)."""
        X = np.ascontiguousarray(X, dtype=np.float32)
        n = X.shape[0]
        out = self._result(n)
        if transposed:
            XT = np.ascontiguousarray(X.T)
            self._check(self._lib.CalcModelPredictionFlatTransposed(self._h, n, _row_pointers(XT), XT.shape[0],
                                                                    out.ctypes.data, out.size))
        elif tree_start or tree_end is not None:
            self._check(self._lib.CalcModelPredictionFlatStaged(self._h, n, tree_start,
                                                                self.tree_count if tree_end is None else tree_end,
                                                                _row_pointers(X), X.shape[1], out.ctypes.data, out.size))
        else:
            self._check(self._lib.CalcModelPredictionFlat(self._h, n, _row_pointers(X), X.shape[1], out.ctypes.data,
                                                          out.size))
        return out

    def predict(self, floats, cats: Sequence[Sequence[str]]) -> np.ndarray:
        """``floats``: float32 [docs][float features]; ``cats``: strings [docs][categorical features]."""
        F = np.ascontiguousarray(floats, dtype=np.float32)
        n = F.shape[0]
        enc = [[str(v).encode("utf-8") for v in row] for row in cats]
        ncat = len(enc[0]) if enc else 0
        rows = [(ctypes.c_char_p * max(1, ncat))(*row) for row in enc]
        cat_ptrs = (ctypes.c_void_p * max(1, n))(*[ctypes.cast(r, ctypes.c_void_p) for r in rows])
        out = self._result(n)
        self._check(self._lib.CalcModelPrediction(self._h, n, _row_pointers(F), F.shape[1] if F.ndim == 2 else 0, cat_ptrs,
                                                  ncat, out.ctypes.data, out.size))
        return out

    def predict_hashed(self, floats, cat_hashes) -> np.ndarray:
        F = np.ascontiguousarray(floats, dtype=np.float32)
        H = np.ascontiguousarray(np.asarray(cat_hashes).astype(np.uint32).view(np.int32))
        n = F.shape[0]
        out = self._result(n)
        self._check(self._lib.CalcModelPredictionWithHashedCatFeatures(self._h, n, _row_pointers(F), F.shape[1],
                                                                       _row_pointers(H), H.shape[1], out.ctypes.data,
                                                                       out.size))
        return out

    def predict_class_flat(self, X, class_id: int) -> np.ndarray:
        X = np.ascontiguousarray(X, dtype=np.float32)
        out = np.empty(X.shape[0], dtype=np.float64)
        self._check(self._lib.PredictSpecificClassFlat(self._h, X.shape[0], _row_pointers(X), X.shape[1], int(class_id),
                                                       out.ctypes.data, out.size))
        return out


def string_cat_hash(s: str) -> int:
    b = s.encode("utf-8")
    return int(library().GetStringCatFeatureHash(b, len(b))) & 0xFFFFFFFF


def integer_cat_hash(v: int) -> int:
    return int(library().GetIntegerCatFeatureHash(int(v))) & 0xFFFFFFFF
