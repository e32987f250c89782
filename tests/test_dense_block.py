"""Single-buffer dense blocks against torchvision's list-and-concatenate blocks (CPU, float64)."""
import copy

import pytest
import torch

tv = pytest.importorskip('torchvision')


def _nets(memory_format):
    from torchvision.models.densenet import DenseNet
    from mgwfbp_b200.models.dense_block import fuse_dense_blocks
    torch.manual_seed(0)
    ref = DenseNet(growth_rate=8, block_config=(3, 4, 2), num_init_features=16, bn_size=2, num_classes=10).double()
    ours = copy.deepcopy(ref)
    assert fuse_dense_blocks(ours) == 3
    ref, ours = ref.to(memory_format=memory_format), ours.to(memory_format=memory_format)
    return ref.train(), ours.train()


@pytest.mark.parametrize('memory_format', [torch.contiguous_format, torch.channels_last])
def test_dense_block_matches_torchvision_forward_and_backward(memory_format):
    ref, ours = _nets(memory_format)
    x = torch.randn(4, 3, 32, 32, dtype=torch.float64).to(memory_format=memory_format)
    y = torch.randint(0, 10, (4,))
    order = {}
    for name, (net, seen) in {'ref': (ref, []), 'ours': (ours, [])}.items():
        for n, p in net.named_parameters():
            p.register_post_accumulate_grad_hook(lambda _p, _n=n, _s=seen: _s.append(_n))
        out = net(x)
        loss = torch.nn.functional.cross_entropy(out, y)
        loss.backward()
        order[name] = (out.detach(), loss.detach(), seen)
    torch.testing.assert_close(order['ours'][0], order['ref'][0], rtol=1e-10, atol=1e-10)
    for (n, a), b in zip(ours.named_parameters(), ref.parameters()):
        torch.testing.assert_close(a.grad, b.grad, rtol=1e-8, atol=1e-10, msg=lambda m, n=n: '%s: %s' % (n, m))
    for (n, a), b in zip(ours.named_buffers(), ref.buffers()):
        torch.testing.assert_close(a, b, rtol=1e-10, atol=1e-12, msg=lambda m, n=n: '%s: %s' % (n, m))
    # every parameter's gradient was delivered exactly once; gradients become ready layer by layer from the back in both
    # (inside one dense layer the two orders may differ, across layers they may not)
    assert sorted(order['ours'][2]) == sorted(order['ref'][2])

    def layer_of(name):
        parts = name.split('.')
        return '.'.join(parts[:3]) if parts[1].startswith('denseblock') else '.'.join(parts[:2])

    def collapse(names):
        out = []
        for n in names:
            k = layer_of(n)
            if not out or out[-1] != k:
                out.append(k)
        return out
    assert collapse(order['ours'][2]) == collapse(order['ref'][2])


def test_dense_block_eval_and_no_grad_use_the_plain_path():
    ref, ours = _nets(torch.contiguous_format)
    x = torch.randn(2, 3, 32, 32, dtype=torch.float64)
    with torch.no_grad():
        torch.testing.assert_close(ours(x), ref(x), rtol=1e-10, atol=1e-10)        # training mode, no graph
    ref.eval(), ours.eval()
    torch.testing.assert_close(ours(x), ref(x), rtol=1e-10, atol=1e-10)


def test_dense_block_two_steps_of_sgd_match():
    ref, ours = _nets(torch.contiguous_format)
    opts = [torch.optim.SGD(n.parameters(), lr=0.05, momentum=0.9) for n in (ref, ours)]
    for step in range(2):
        x = torch.randn(4, 3, 32, 32, dtype=torch.float64)
        y = torch.randint(0, 10, (4,))
        for net, opt in zip((ref, ours), opts):
            opt.zero_grad()
            torch.nn.functional.cross_entropy(net(x), y).backward()
            opt.step()
    for (n, a), b in zip(ours.named_parameters(), ref.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-8, atol=1e-10, msg=lambda m, n=n: '%s: %s' % (n, m))


def test_fused_forwards_follow_the_module_through_replication():
    """nn.DataParallel replicates modules by copying their __dict__: a rebound forward has to live on the class, or every
    replica would run the original module's forward (on the original's parameters)."""
    from mgwfbp_b200.models.fuse import fuse_model
    net = fuse_model(tv.models.densenet121(num_classes=10))
    for m in (net.features.denseblock1, net.features.denseblock1.denselayer1, net):
        rep = m._replicate_for_data_parallel()
        assert rep.forward.__self__ is rep
        assert 'forward' not in m.__dict__
    assert isinstance(net.features.denseblock1, tv.models.densenet._DenseBlock)
    fuse_model(net)                                       # idempotent: no second layer of subclasses
    assert type(net.features.denseblock1).__mro__[1] is tv.models.densenet._DenseBlock


def test_dense_block_under_autocast():
    """Mixed precision: layers may produce a narrower type than the block buffer holds; forward and backward still run
    and agree with the list-and-concatenate path to the precision of the narrow type."""
    import copy
    from torchvision.models.densenet import DenseNet
    from mgwfbp_b200.models.dense_block import fuse_dense_blocks
    torch.manual_seed(0)
    ref = DenseNet(growth_rate=8, block_config=(3, 2), num_init_features=16, bn_size=2, num_classes=10).train()
    ours = copy.deepcopy(ref)
    fuse_dense_blocks(ours)
    x = torch.randn(4, 3, 32, 32)
    y = torch.randint(0, 10, (4,))
    losses = []
    for net in (ref, ours):
        with torch.autocast('cpu', dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(net(x).float(), y)
        loss.backward()
        losses.append(float(loss.detach()))
    assert abs(losses[0] - losses[1]) < 5e-2
    for (n, a), b in zip(ours.named_parameters(), ref.parameters()):
        assert a.grad is not None and a.grad.dtype == b.grad.dtype and torch.isfinite(a.grad).all(), n
    ga = torch.cat([p.grad.flatten() for p in ours.parameters()])
    gb = torch.cat([p.grad.flatten() for p in ref.parameters()])
    assert float((ga - gb).norm() / gb.norm()) < 0.2          # bfloat16 layers: same gradient up to the type's noise


def test_row_layout_accepts_only_what_the_strided_kernels_can_read():
    """The BatchNorm kernels read ``x[r * ld + c]``: a dense channels-innermost tensor, or the channels ``[a, a + C)`` of a
    wider channels-last tensor over ALL of its pixels (any batch range).  Everything else must be refused (and is then
    copied), because nothing on the device checks the layout."""
    from mgwfbp_b200.ops.bn_relu import _row_layout
    w = torch.empty(4, 64, 8, 8).contiguous(memory_format=torch.channels_last)
    assert _row_layout(w) == (256, 64, 64)
    assert _row_layout(w[:, :32]) == (256, 32, 64)                  # leading channels
    assert _row_layout(w[:, 4:36]) == (256, 32, 64)                 # 16-byte aligned channel offset
    assert _row_layout(w[1:3, :32]) == (128, 32, 64)                # a batch range keeps rows equidistant
    assert _row_layout(w[:, :30]) == (256, 30, 64)                  # scalar path: no alignment rule on C
    assert _row_layout(w[:, 1:33]) is None                          # vector path at a 4-byte offset
    assert _row_layout(w[:, :32, :4]) is None                       # rows of different images are not equidistant
    assert _row_layout(w[:, :32, :, :4]) is None
    assert _row_layout(w[:, :32, ::2]) is None
    assert _row_layout(torch.empty(4, 64, 8, 8)) is None            # NCHW
    assert _row_layout(torch.empty(4, 64, 8, 8)[:, :32]) is None
    assert _row_layout(torch.empty(4, 64, 8, 1).contiguous(memory_format=torch.channels_last)[:, :32]) is None   # W = 1
    odd = torch.empty(4, 66, 8, 8).contiguous(memory_format=torch.channels_last)
    assert _row_layout(odd[:, :32]) is None                         # row stride 66: rows are not 16-byte aligned
    assert _row_layout(odd[:, :33]) == (256, 33, 66)
    two_d = torch.empty(16, 12)
    assert _row_layout(two_d) == (16, 12, 12) and _row_layout(two_d[:, :8]) is None
