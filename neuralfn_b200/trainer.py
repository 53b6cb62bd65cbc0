"""Scalar-graph edge trainers under their reference names (``neuralfn/trainer.py``):
``SurrogateTrainer`` / ``TrainConfig`` (Adam through frozen surrogates) plus the exact
gradient ``GraphSGDTrainer`` this framework adds."""
from .sgd import GraphSGDTrainer, SGDConfig, init_edge_params_normal  # noqa: F401
from .surrogate import SurrogateTrainer, TrainConfig  # noqa: F401
