"""Epilogue selectors accepted by the `epilogue=` argument (csrc/apis/epilogue_class.hpp:10-21)."""

from ._api import Alpha, BF16StochasticRounding, Epilogue, FP8Quantization, Identity  # noqa: F401
