"""archlab-b200: a Blackwell-native architecture-research training framework.

Public entry points: ``archlab_b200.cli:main`` (``archlab {resolve|qualify|train}``),
``archlab_b200.train.speedrun.Trainer`` (pre-training step API), ``archlab_b200.ops`` (sm_100a
kernels with PyTorch reference statements) and ``archlab_b200.models`` (model zoo).
"""

__version__ = "0.1.0"
