"""``MyAutogradFunc`` — the contract every operator class of this layer implements.

Follows the contract that intrasm_engine/pytorch/cpp_extensions/layers_and_funcs/utils.py:11-144
documents: ``_forward(*args, **fwd_kwargs) -> (outputs, ctx_dict, tensors_to_save)`` and
``_backward(*grads, *saved_tensors, **ctx_dict) -> grads``, so that two or three operators
can run as ONE autograd node that saves tensors once.  ``torch.autograd.Function.apply``
takes no keyword arguments, so the per-operator keyword dictionaries travel as the first
positional argument; ``cls.run(*args, fwd_kwargs_1={...})`` packs them.
"""
from __future__ import annotations

from typing import Any, Optional

import torch

# Keyword arguments every ``_forward`` receives (sputnik.py:48-53, torch.py:10-15).
FWD_KWARG_NAMES = ("constructor", "backward_constructor", "num_streams", "constructor_enabled",
                   "stream_beg")


def default_fwd_kwargs(**overrides) -> dict:
    kw = {"constructor": None, "backward_constructor": None, "num_streams": 1,
          "constructor_enabled": False, "stream_beg": 0}
    kw.update(overrides)
    return kw


def assert_params_unpacked(params: dict):
    for key in params:
        assert not key.startswith("space_")


class captured:
    """``with captured(constructor, stream_idx, enabled):`` records the enclosed library
    calls into the constructor's graph on its registered stream ``stream_idx`` — the
    bracket the reference writes out around every op call (sputnik.py:58-66)."""

    def __init__(self, constructor, stream_idx: int, enabled: bool):
        # no constructor to record into (e.g. a backward pass without a backward constructor):
        # the enclosed calls simply run
        self.constructor, self.stream_idx = constructor, stream_idx
        self.enabled = bool(enabled) and constructor is not None
        self._stream = None

    def __enter__(self):
        if self.enabled:
            self._stream = self.constructor.registeredStreams[self.stream_idx]
            self._stream.__enter__()
            self.constructor.capture_library_call_begin()
        return self

    def __exit__(self, *exc):
        if self.enabled:
            try:
                self.constructor.capture_library_call_end()
            finally:
                self._stream.__exit__(*exc)
        return False


class MyAutogradFunc(torch.autograd.Function):
    @staticmethod
    def num_inputs(**fwd_kwargs_unwrapped) -> int:
        raise NotImplementedError("You must implement num_inputs for your autograd function.")

    @staticmethod
    def num_outputs(**ctx_kwargs_unwrapped) -> int:
        raise NotImplementedError("You must implement num_outputs for your autograd function.")

    @staticmethod
    def num_saved_tensors(**ctx_kwargs_unwrapped) -> int:
        raise NotImplementedError("You must implement num_saved_tensors for your autograd function.")

    @staticmethod
    def _forward(*args, **fwd_kwargs_unwrapped
                 ) -> tuple[tuple[torch.Tensor, ...], dict, tuple[torch.Tensor, ...]]:
        """Returns (outputs, dictionary to keep for backward, tensors to save)."""
        raise NotImplementedError("You must implement _forward for your autograd function.")

    @staticmethod
    def _backward(*grad_and_saved_tensors, **ctx_kwargs_unwrapped) -> tuple:
        """Takes ``*grads, *saved_tensors, **ctx_dict``; returns one gradient per input."""
        raise NotImplementedError("You must implement _backward for your autograd function.")

    @classmethod
    def run(cls, *args, **fwd_kwargs):
        """``apply`` with keyword dictionaries (``fwd_kwargs_1=...``; defaults when omitted).
        A class that has not been through ``make_single_kernel_autograd_function`` yet (the
        factory of horizontal_rewriter that builds ``forward`` / ``backward`` from ``_forward`` /
        ``_backward``) is put through it here, so that ``run`` works whatever was imported first."""
        if "forward" not in cls.__dict__:
            from ....pytorch.horizontal_rewriter import make_single_kernel_autograd_function
            make_single_kernel_autograd_function(cls)
        if not fwd_kwargs:
            fwd_kwargs = {"fwd_kwargs_1": default_fwd_kwargs()}
        return cls.apply(fwd_kwargs, *args)

    # -- tuning interface of the reference (utils.py:71-144); no tuner ships here ----------
    @classmethod
    def get_search_space(cls, sample_inputs: list, sample_grads: Optional[list]) -> dict:
        return {}

    @classmethod
    def _check_unwrapped_fwd_kwargs_sanity(cls, unwrapped_fwd_kwargs: dict[str, Any]):
        for name in FWD_KWARG_NAMES:
            assert name in unwrapped_fwd_kwargs, f"missing forward kwarg {name}"
        assert unwrapped_fwd_kwargs["num_streams"] == 1

    @classmethod
    def check_fwd_kwargs_sanity(cls, fwd_kwargs: dict[str, Any]):
        assert "fwd_kwargs_1" in fwd_kwargs
        return cls._check_unwrapped_fwd_kwargs_sanity(fwd_kwargs["fwd_kwargs_1"])

    @classmethod
    def check_params_sanity(cls, params: dict):
        assert_params_unpacked(params)

    @classmethod
    def get_test_fwd_kwargs(cls, params: dict) -> dict[str, Any]:
        return {"fwd_kwargs_1": default_fwd_kwargs(**params)}

    @classmethod
    def build_and_test(cls, sample_inputs: list, sample_grads: Optional[list], params: dict):
        """One forward and backward through ``_forward`` / ``_backward`` with the given point
        of the search space; returns ``(outputs, grad_inputs)``."""
        kw = cls.get_test_fwd_kwargs(params)["fwd_kwargs_1"]
        outputs, ctx_dict, saved = cls._forward(*sample_inputs, **kw)
        if sample_grads is None:
            sample_grads = tuple(torch.randn_like(o) for o in outputs)
        grads = cls._backward(*sample_grads, *saved, **ctx_dict)
        return outputs, grads
