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
