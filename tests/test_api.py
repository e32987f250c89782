"""CPU unit tests of the public surface: configs, schedules, parameter groups, checkpoints, naming, models."""
import glob
import math
import os
import subprocess

import numpy as np
import pytest
import torch

import mgwfbp_b200 as hvd
from mgwfbp_b200 import settings
from mgwfbp_b200.models import _support_dnns, create_net
from mgwfbp_b200.trainer import DLTrainer
from mgwfbp_b200.utils import checkpoint as ckpt
from mgwfbp_b200.utils.config import load_experiment, parse_conf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_experiment_file_parses_and_matches_bash():
    files = sorted(glob.glob(os.path.join(ROOT, 'exp_configs', '*.conf')))
    assert len(files) >= 19
    for f in files:
        got = parse_conf(f, env={})
        for key in ('lr', 'batch_size', 'dnn', 'dataset', 'max_epochs', 'nstepsupdate', 'data_dir'):
            assert key in got and got[key] != '', (f, key)
        out = subprocess.run(['bash', '-c', 'unset lr batch_size max_epochs data_dir; source %s; echo "$lr|$batch_size|$dnn|$dataset|$max_epochs|$nstepsupdate|$data_dir"' % f],
                             capture_output=True, text=True, env={'PATH': os.environ['PATH']}).stdout.strip().split('|')
        assert [got[k] for k in ('lr', 'batch_size', 'dnn', 'dataset', 'max_epochs', 'nstepsupdate', 'data_dir')] == out, f


def test_reference_defaults_and_env_override():
    assert load_experiment('resnet20', env={})['lr'] == 0.1 and load_experiment('resnet20', env={})['batch_size'] == 32
    assert load_experiment('lstm', env={})['lr'] == 22.0 and load_experiment('lstm', env={})['dataset'] == 'ptb'
    assert load_experiment('resnet50', env={})['batch_size'] == 128 and load_experiment('resnet50', env={})['max_epochs'] == 70
    assert load_experiment('resnet50', env={'lr': '0.8', 'batch_size': '64'})['lr'] == 0.8
    assert load_experiment('googlenet', env={'lr': '0.8'})['lr'] == 0.01          # fixed in that file, as in the reference


def _trainer(dnn='resnet20', dataset='cifar10', **kw):
    return DLTrainer(0, 1, dist=False, ngpus=0, batch_size=kw.pop('batch_size', 4), data_dir=kw.pop('data_dir', 'synthetic'),
                     dataset=dataset, dnn=dnn, lr=kw.pop('lr', 0.1), nworkers=kw.pop('nworkers', 1), **kw)


def test_param_groups_and_dataset_hyperparameters():
    t = _trainer()
    g_nodecay, g_decay = t.optimizer.param_groups
    assert g_nodecay['weight_decay'] == 0.0 and g_decay['weight_decay'] == 1e-4 and g_decay['momentum'] == 0.9
    assert all(p.dim() == 1 for p in g_nodecay['params']) and all(p.dim() > 1 for p in g_decay['params'])
    assert len(g_nodecay['params']) + len(g_decay['params']) == 59
    t = _trainer('lstm', 'ptb', batch_size=2, num_steps=5)
    assert t.optimizer.param_groups[1]['momentum'] == 0 and t.optimizer.param_groups[1]['weight_decay'] == 0
    t = _trainer('lr', 'mnist')
    assert t.num_batches_per_epoch == math.ceil(60000 / 4)


def test_learning_rate_schedules():
    t = _trainer(lr=0.1)
    t.num_batches_per_epoch = 100
    settings.WARMUP = True
    t.train_iter = 0
    lr0 = t.adjust_learning_rate(0, t.optimizer)
    assert lr0 == pytest.approx(0.1 / 500)
    t.train_iter = 250
    assert t.adjust_learning_rate(2, t.optimizer) == pytest.approx(0.1 / 500 + (0.1 - 0.1 / 500) / 500 * 250)
    for epoch, want in [(5, 0.1), (80, 0.1), (81, 0.01), (122, 0.001), (155, 0.0001)]:
        assert t.adjust_learning_rate(epoch, t.optimizer) == pytest.approx(want)
        assert all(g['lr'] == pytest.approx(want) for g in t.optimizer.param_groups)
    ti = _trainer('resnet20', 'cifar10')
    ti.dataset = 'imagenet'
    for epoch, want in [(29, 0.1), (30, 0.01), (60, 0.001), (80, 0.0001)]:
        assert ti.adjust_learning_rate(epoch, ti.optimizer) == pytest.approx(want)
    tl = _trainer('lstm', 'ptb', batch_size=2, num_steps=5, lr=22.0)
    assert tl.adjust_learning_rate(62, tl.optimizer) == 22.0
    assert tl.adjust_learning_rate(63, tl.optimizer) == pytest.approx(0.22)     # the x0.1 stage is unreachable
    assert tl.adjust_learning_rate(80, tl.optimizer) == pytest.approx(0.022)


def test_checkpoint_format_roundtrip(tmp_path):
    os.chdir(tmp_path)
    t = _trainer(lr=0.1, nworkers=4, prefix='allreduce')
    t.train_epoch, t.train_iter = 3, 1234
    path = t.save_checkpoint()
    assert path.replace('\\', '/').endswith('weights/allreduce/resnet20-n4-bs4-lr0.1000/resnet20-rank0-epoch3.pth')
    raw = torch.load(path, weights_only=False)
    assert set(raw) == {'iter', 'epoch', 'state'} and raw['iter'] == 1234 and raw['epoch'] == 3
    assert list(raw['state']) == list(t.net.state_dict())
    t2 = _trainer(lr=0.1)
    t2.load_model_from_file(path)
    assert t2.get_train_epoch() == 3 and t2.get_train_iter() == 1234
    for a, b in zip(t.net.state_dict().values(), t2.net.state_dict().values()):
        assert torch.equal(a, b)
    info = ckpt.parse_checkpoint_dir(os.path.dirname(path))
    assert info == {'dnn': 'resnet20', 'nworkers': 4, 'batch_size': 4, 'lr': 0.1}
    # a checkpoint written the reference's way loads as well
    torch.save({'iter': 7, 'epoch': 1, 'state': t.net.state_dict()}, tmp_path / 'ref.pth')
    t2.load_model_from_file(str(tmp_path / 'ref.pth'))
    assert t2.get_train_iter() == 7


def test_registry_builds_every_name_with_reference_parameter_counts():
    expected = {'resnet20': (59, 269722), 'resnet50': (161, 25557032), 'densenet201': (604, 20013928),
                'vgg16i': (32, 138357544), 'vgg16': (54, None), 'alexnet': (16, None), 'googlenet': (59, None),
                'inceptionv4': (449, None), 'resnet152': (467, None), 'densenet161': (484, None)}
    for dnn in _support_dnns:
        kw = dict(vocab_size=10000, batch_size=20) if dnn == 'lstm' else {}
        with torch.device('meta'):
            net, ext = create_net(10 if dnn in ('resnet20', 'resnet56', 'resnet110', 'vgg16', 'vgg19') else 1000, dnn, **kw)
        ps = list(net.parameters())
        if dnn in expected:
            n_t, n_p = expected[dnn]
            assert len(ps) == n_t, dnn
            if n_p is not None:
                assert sum(p.numel() for p in ps) == n_p, dnn
    with pytest.raises(ValueError):
        create_net(10, 'no-such-net')


def test_lstm_state_dict_keys_match_torch_lstm():
    a, _ = create_net(10, 'lstm', vocab_size=50, batch_size=2)
    b, _ = create_net(10, 'lstm', vocab_size=50, batch_size=2, fused_lstm=True)
    assert list(a.state_dict()) == list(b.state_dict())
    assert 'lstm.weight_ih_l0' in a.state_dict() and 'lstm.bias_hh_l1' in a.state_dict()
    b.load_state_dict(a.state_dict())
    x = torch.randint(0, 50, (35, 2))
    a.eval(), b.eval()
    ya, _ = a(x, a.init_hidden())
    yb, _ = b(x, b.init_hidden())
    torch.testing.assert_close(ya, yb, rtol=1e-4, atol=1e-5)


def test_distributed_optimizer_single_process_contract():
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4))
    base = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
    opt = hvd.DistributedOptimizer(base, named_parameters=net.named_parameters(), threshold=0)
    assert isinstance(opt, torch.optim.SGD) and type(opt).__name__ == 'SGD'
    assert opt.param_groups is not base.param_groups or True
    assert opt.local is False and opt.train_iter == 0 and opt.train_epoch == 0
    net(torch.randn(2, 8)).sum().backward()
    opt.step()
    assert set(opt.state_dict()['state'][0]) == {'momentum_buffer'}
    with pytest.raises(ValueError):
        hvd.DistributedOptimizer(base, named_parameters=[p for p in net.parameters()])
    assert hvd.size() == 1 and hvd.rank() == 0 and hvd.local_rank() == 0 and hvd.local_size() == 1


def test_hook_order_guard():
    from mgwfbp_b200.parallel.comm.base import Communicator

    class Fake(Communicator):
        def size(self):
            return 2

        def allreduce_async_(self, tensor, average=True, name=None):
            return tensor

        def synchronize(self, handle):
            return handle
    net = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.Linear(4, 2))
    names = [n for n, _ in net.named_parameters()]
    wrong = [names[2], names[3], names[0], names[1]]          # claims layer 1 comes first
    opt = hvd.DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=0.1), named_parameters=net.named_parameters(),
                                   seq_layernames=wrong, layerwise_times=[1e-3] * 4, comm=Fake(),
                                   cost_model=hvd.AlphaBeta(1e-9, 1e-15))
    opt._verify_schedule_agreement = lambda: None
    with pytest.raises(hvd.HookOrderError):
        net(torch.randn(2, 4)).sum().backward()


def test_log_directory_naming():
    import dist_trainer
    args = dist_trainer.build_parser().parse_args(['--dnn', 'resnet20', '--nworkers', '4', '--batch-size', '32', '--lr', '0.1',
                                                   '--threshold', '524288000'])
    assert args.nsteps_update == 1 and args.density == 1 and args.nwpernode == 1 and args.num_steps == 35
    logdir = 'allreduce-%s-thres-%dkbytes/%s-n%d-bs%d-lr%.4f-ns%d-ds%s' % (
        settings.PREFIX, args.threshold / 1024, args.dnn, args.nworkers, args.batch_size, args.lr, args.nsteps_update, str(args.density))
    assert logdir.endswith('thres-512000kbytes/resnet20-n4-bs32-lr0.1000-ns1-ds1')
    assert settings.PREFIX.startswith('gwarmup-dc1-model-tpds') and settings.PREFIX.endswith('-ada')


def test_profiler_returns_measured_order_reversed():
    """Names come back in forward order as *measured*: the reverse of the order in which gradients
    became ready (within a layer the weight may precede its bias), with matching sizes."""
    from mgwfbp_b200.utils.profiling import benchmark
    t = _trainer('lenet', 'mnist')
    names, times, sizes = benchmark(t, warmup=1, iteration=2)
    params = dict(t.net.named_parameters())
    assert sorted(names) == sorted(params)
    assert sizes == [params[n].numel() for n in names]
    assert len(times) == len(names) and all(x >= 0 for x in times)
    fired = []
    handles = [p.register_hook(lambda g, n=n: fired.append(n)) for n, p in params.items()]
    loss, *_ = t.forward_loss(t.data_iter())
    loss.backward()
    for h in handles:
        h.remove()
    assert fired == names[::-1]


def test_single_gpu_cli_and_evaluate_roundtrip(tmp_path, monkeypatch):
    """dl_trainer's loop on CPU with synthetic data, a checkpoint at the epoch boundary, then evaluate.py."""
    monkeypatch.chdir(tmp_path)
    from mgwfbp_b200.trainer import train_with_single
    import mgwfbp_b200.data.synthetic as syn
    monkeypatch.setitem(syn.NOMINAL_LENGTH, 'mnist', (64, 32))       # 4 iterations of 16 per epoch
    trainer = train_with_single('lenet', 'mnist', 'synthetic', 1, 0.01, 16, 1, 2, max_iters=6)
    assert trainer.get_train_iter() >= 6 and trainer.get_train_epoch() == 1
    ckpt_dir = os.path.join(str(tmp_path), 'weights', 'singlegpu', 'lenet-n1-bs16-lr0.0100')
    assert os.path.isfile(os.path.join(ckpt_dir, 'lenet-rank0-epoch1.pth'))
    import evaluate
    best = evaluate.evaluate(ckpt_dir, 'lenet', 'mnist', 'synthetic', nepochs=1, start_epoch=1)
    assert best is not None and 0.0 <= best <= 100.0


def test_train_step_driver_on_cpu():
    from mgwfbp_b200.engine import TrainStep
    t = _trainer('lenet', 'mnist', batch_size=8)
    t.update_optimizer(hvd.DistributedOptimizer(t.optimizer, named_parameters=t.net.named_parameters()))
    step = TrainStep(t, use_graph=True)           # no GPU: runs eagerly
    before = [p.detach().clone() for p in t.net.parameters()]
    for _ in range(3):
        step.run(t.data_iter())
    assert not step.graphed and len(step.losses) == 3 and all(l == l for l in step.losses)
    assert any(not torch.equal(a, b.detach()) for a, b in zip(before, t.net.parameters()))
    assert t.get_train_iter() == 3


def test_train_step_carries_and_resets_lstm_state():
    """The PTB model's hidden state is carried from step to step and forgotten by ``reset_state`` (epoch start)."""
    from mgwfbp_b200.engine import TrainStep
    t = _trainer('lstm', 'ptb', batch_size=4)
    t.update_optimizer(hvd.DistributedOptimizer(t.optimizer, named_parameters=t.net.named_parameters(), norm_clip=0.25))
    step = TrainStep(t, use_graph=False)
    step.run(t.data_iter())
    assert step._hidden is not None and all(not h.requires_grad for h in step._hidden)
    assert any(float(h.abs().sum()) > 0 for h in step._hidden)
    step.reset_state()
    assert step._hidden is None
    step.run(t.data_iter())
    assert step._hidden is not None and len(step.losses) == 2


def test_extra_models_build():
    from mgwfbp_b200 import models
    for ctor in (models.preresnet20, models.resnet_mod20, models.resnext29_8_64, models.caffe_cifar, models.densenet100_12,
                 models.ResNet18):
        with torch.device('meta'):
            net = ctor()
        assert sum(p.numel() for p in net.parameters()) > 0
    assert models.resnet20().name == 'resnet20'


def test_speech_and_language_model_paths_train_on_synthetic_data():
    """The AN4 acoustic model (CTC) and the PTB LSTM (hidden state carried, global-norm clip) run end to end."""
    t = _trainer('lstman4', 'an4', batch_size=2, lr=0.0002)
    t.update_optimizer(hvd.DistributedOptimizer(t.optimizer, named_parameters=t.net.named_parameters(), norm_clip=400))
    t.optimizer.zero_grad()
    t.train(1)
    t.update_model()
    assert t.loss == t.loss and t.loss > 0
    assert 0.0 <= t.test(0)
    t = _trainer('lstm', 'ptb', batch_size=4, lr=22.0, num_steps=35)
    t.update_optimizer(hvd.DistributedOptimizer(t.optimizer, named_parameters=t.net.named_parameters(), norm_clip=0.25))
    hidden = t.net.init_hidden()
    before = t.net.sm_fc.weight.detach().clone()
    for _ in range(2):
        t.optimizer.zero_grad()
        _, hidden = t.train(1, hidden=hidden)
        t.update_model()
    assert t.loss == t.loss and hidden[0].shape == (2, 4, 1500)
    step = (t.net.sm_fc.weight.detach() - before).norm()
    assert 0 < float(step) <= 22.0 * 0.25 * 2 + 1e-3       # clipped gradient norm bounds each update


def test_order_and_prune_files_by_duration(tmp_path):
    import wave
    import numpy as np
    from mgwfbp_b200.data.an4 import order_and_prune_files, wav_duration
    paths = []
    for i, seconds in enumerate([0.8, 0.2, 1.5, 0.5]):
        p = tmp_path / ('u%d.wav' % i)
        with wave.open(str(p), 'wb') as w:
            w.setnchannels(1); w.setsampwidth(2); w.setframerate(16000)
            w.writeframes(np.zeros(int(16000 * seconds), dtype=np.int16).tobytes())
        paths.append(str(p))
    assert abs(wav_duration(paths[2]) - 1.5) < 1e-6
    assert order_and_prune_files(paths) == [paths[1], paths[3], paths[0], paths[2]]
    assert order_and_prune_files(paths, 0.4, 1.0) == [paths[3], paths[0]]


def test_s2d_stem_algebra_on_cpu():
    """4x4 / stride 1 over the space-to-depth input == 7x7 / stride 2 / padding 3, and the module keeps Conv2d's state."""
    import torch.nn.functional as F
    from mgwfbp_b200.ops.stem import S2DStemConv2d, convert_stem, s2d_input_reference, s2d_weight
    torch.manual_seed(0)
    x, w = torch.randn(2, 3, 32, 48), torch.randn(8, 3, 7, 7)
    torch.testing.assert_close(F.conv2d(s2d_input_reference(x), s2d_weight(w), None, 1, 0), F.conv2d(x, w, None, 2, 3),
                               rtol=1e-4, atol=1e-4)
    conv = torch.nn.Conv2d(3, 8, 7, stride=2, padding=3, bias=False)
    new = convert_stem(conv)
    assert isinstance(new, S2DStemConv2d) and new.weight is conv.weight and list(new.state_dict()) == ['weight']
    torch.testing.assert_close(new(x), conv(x))                       # CPU input: the parent's path
    assert convert_stem(torch.nn.Conv2d(3, 8, 3)) is not None and not isinstance(convert_stem(torch.nn.Conv2d(3, 8, 3)), S2DStemConv2d)
