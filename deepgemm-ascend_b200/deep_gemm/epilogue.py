"""Epilogue selectors accepted by the `epilogue=` argument (csrc/apis/epilogue_class.hpp:10-21): the classes of the
compiled `_C` extension when it is built, else those of the Python host layer."""

from . import _api

if _api._C is not None:
    Epilogue = _api._C.epilogue.Epilogue
    Identity = _api._C.epilogue.Identity
    Alpha = _api._C.epilogue.Alpha
    FP8Quantization = _api._C.epilogue.FP8Quantization
    BF16StochasticRounding = _api._C.epilogue.BF16StochasticRounding
else:
    from ._api import Alpha, BF16StochasticRounding, Epilogue, FP8Quantization, Identity  # noqa: F401
