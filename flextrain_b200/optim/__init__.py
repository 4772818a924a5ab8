"""Optimizers: AdamW, Muon and the per-tensor hybrid (flextrain/optim/*.py).

An optimizer is stateless apart from its hyper-parameters; the engine owns the state tensors
(so they can live in HBM, in pinned host memory or in a data-parallel shard) and hands them in:

    code = opt.step(param_spec, params, grads, state, step_num, grad_scale=1.0)

State keys follow flextrain/optim/base.py:77-87: ``o_adam_m_<suffix>``, ``o_adam_v_<suffix>``,
``o_muon_<suffix>`` where ``w_q -> q``.  ``step`` returns non-zero when ``check_error`` finds a
NaN/Inf gradient, in which case nothing was updated.
"""
from .adamw import AdamW, AdamWHyperparams
from .base import Optimizer, OptimizerStateSpec, OptStateTensor, ReferenceStyleOptimizer, as_engine_optimizer, state_key
from .hybrid import HybridMuonAdamW, HybridMuonAdamWHyperparams, infer_optimizer_for_param, uses_muon
from .muon import Muon, MuonHyperparams

__all__ = ["AdamW", "AdamWHyperparams", "HybridMuonAdamW", "HybridMuonAdamWHyperparams", "Muon", "MuonHyperparams",
           "OptStateTensor", "Optimizer", "OptimizerStateSpec", "ReferenceStyleOptimizer", "as_engine_optimizer",
           "infer_optimizer_for_param", "state_key", "uses_muon"]
