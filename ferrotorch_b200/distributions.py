"""Probability distributions, KL registry, transforms and constraints: ``torch.distributions``
re-exported (the reference's ``ferrotorch-distributions`` mirrors that package: 30 distributions,
``kl``, ``transforms``, ``constraints``)."""
from torch.distributions import *  # noqa: F401,F403
from torch.distributions import constraints, kl, transforms  # noqa: F401
from torch.distributions.kl import kl_divergence, register_kl  # noqa: F401
from torch.distributions.constraints import Constraint as DistConstraint  # noqa: F401,E402
from torch.distributions.relaxed_categorical import ExpRelaxedCategorical  # noqa: F401,E402


def kl_expfamily_expfamily(p, q):
    """KL(p || q) of two members of the same exponential family as the Bregman divergence of
    the log-normaliser, ``A(eta_q) - A(eta_p) - <eta_q - eta_p, grad A(eta_p)>`` (exp_family.rs:71;
    the gradient comes from autograd here, the reference writes it in closed form)."""
    import torch

    if type(p) is not type(q):
        raise NotImplementedError("kl_expfamily_expfamily: operands must belong to the same family (%s vs %s)"
                                  % (type(p).__name__, type(q).__name__))
    pn = [t.detach().requires_grad_() for t in p._natural_params]
    qn = q._natural_params
    lg_p = p._log_normalizer(*pn)
    grads = torch.autograd.grad(lg_p.sum(), pn, create_graph=True)
    out = q._log_normalizer(*qn) - lg_p
    for a, b, g in zip(pn, qn, grads):
        term = (b - a) * g
        out = out - (term if term.dim() == out.dim() else term.reshape(out.shape + (-1,)).sum(-1))
    return out.detach() if not any(t.requires_grad for t in qn) else out


# constraint constructors and instances at the top level, as the reference's crate exposes them (constraints.rs)
from torch.distributions.constraints import (boolean, corr_cholesky, greater_than, greater_than_eq, half_open_interval,  # noqa: F401,E402
                                             integer_interval, less_than, lower_cholesky, nonnegative, nonnegative_integer,
                                             positive, real, real_vector, simplex, unit_interval)
from torch.distributions.constraints import interval as closed_interval  # noqa: F401,E402


class _OpenInterval(constraints.Constraint):
    """``lower < x < upper``."""

    def __init__(self, lower_bound, upper_bound):
        self.lower_bound, self.upper_bound = lower_bound, upper_bound
        super().__init__()

    def check(self, value):
        return (self.lower_bound < value) & (value < self.upper_bound)

    def __repr__(self):
        return "open_interval(lower_bound=%s, upper_bound=%s)" % (self.lower_bound, self.upper_bound)


open_interval = _OpenInterval


def try_kl_expfamily(p, q):
    """``KL(p || q)`` through the exponential-family formula when both operands belong to the same family that
    defines natural parameters and a log-normaliser, else ``None`` (exp_family.rs:164)."""
    if type(p) is not type(q) or not isinstance(p, ExponentialFamily):  # noqa: F405
        return None
    try:
        return kl_expfamily_expfamily(p, q)
    except NotImplementedError:
        return None


def kl_divergence_dyn(p, q):
    """``KL(p || q)`` for operands whose types are only known at run time: the registered closed form when
    there is one, else the exponential-family formula, else an error (kl.rs ``kl_divergence_dyn``)."""
    try:
        return kl_divergence(p, q)
    except NotImplementedError:
        out = try_kl_expfamily(p, q)
        if out is None:
            raise
        return out
