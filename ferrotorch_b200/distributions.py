"""Probability distributions, KL registry, transforms and constraints: ``torch.distributions``
re-exported (the reference's ``ferrotorch-distributions`` mirrors that package: 30 distributions,
``kl``, ``transforms``, ``constraints``)."""
from torch.distributions import *  # noqa: F401,F403
from torch.distributions import constraints, kl, transforms  # noqa: F401
from torch.distributions.kl import kl_divergence, register_kl  # noqa: F401
