"""Shadow-path arithmetic (CPU): the written-out SGD update against torch.optim.SGD, and the checker on a stand-in optimizer."""
import types

import pytest
import torch

from mgwfbp_b200.utils.consistency import ShadowChecker, ShadowMismatchError, reference_sgd_update


@pytest.mark.parametrize('momentum,dampening,nesterov,wd', [(0.0, 0.0, False, 0.0), (0.9, 0.0, False, 1e-4), (0.9, 0.0, True, 5e-4),
                                                           (0.8, 0.1, False, 0.0)])
def test_reference_update_is_torch_sgd(momentum, dampening, nesterov, wd):
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(37, 5))
    opt = torch.optim.SGD([p], lr=0.1, momentum=momentum, dampening=dampening, nesterov=nesterov, weight_decay=wd)
    w, buf = p.detach().clone(), None
    for it in range(4):
        g = torch.randn(37, 5)
        p.grad = g.clone()
        opt.step()
        w, buf = reference_sgd_update(w, g, buf, 0.1, wd, momentum, dampening, nesterov, first_step=(it == 0))
        torch.testing.assert_close(w, p.detach(), rtol=1e-6, atol=1e-7)


def _stand_in(clip=None):
    torch.manual_seed(1)
    p = torch.nn.Parameter(torch.randn(50))
    q = torch.nn.Parameter(torch.randn(3, 7))
    base = torch.optim.SGD([{'params': [p], 'weight_decay': 1e-3}, {'params': [q], 'weight_decay': 0.0}], lr=0.2, momentum=0.9)
    fake = types.SimpleNamespace(_named_parameters={'p': p, 'q': q}, state=base.state, param_groups=base.param_groups,
                                 _norm_clip=clip, train_iter=0)
    return fake, base, p, q


@pytest.mark.parametrize('clip', [None, 0.5])
def test_checker_follows_torch_sgd_and_flags_a_wrong_update(clip):
    fake, base, p, q = _stand_in(clip)
    chk = ShadowChecker(every=1)
    for it in range(3):
        p.grad, q.grad = torch.randn(50), torch.randn(3, 7)
        chk.snapshot(fake, ['q', 'p'], first_step=(it == 0))
        if clip is not None:
            torch.nn.utils.clip_grad_norm_([p, q], clip)
        base.step()
        assert chk.verify(fake) == 2
    p.grad, q.grad = torch.randn(50), torch.randn(3, 7)
    chk.snapshot(fake, ['q', 'p'], first_step=False)
    if clip is not None:
        torch.nn.utils.clip_grad_norm_([p, q], clip)
    base.step()
    with torch.no_grad():
        p[17] += 1e-2                                  # what a kernel that mis-addressed one element would leave
    with pytest.raises(ShadowMismatchError, match="parameter p "):
        chk.verify(fake)
    assert chk.verify(fake) == 0                       # snapshots are consumed either way
