"""Merge-schedule tests: golden vectors and equivalence with the reference's own grouping code."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from mgwfbp_b200.parallel.costmodel import (AlphaBeta, PiecewiseAlphaBeta, TABLE_10GBE, TABLE_56GBIB, fit_alpha_beta,
                                            fit_piecewise, table_lookup)
from mgwfbp_b200.parallel.scheduler import check_unique, groups_by_threshold, groups_mgwfbp, simulate_schedule

HERE = os.path.dirname(os.path.abspath(__file__))

TOY_NAMES = ['0.weight', '0.bias', '1.weight', '1.bias', '2.weight', '2.bias', '3.weight', '3.bias']
TOY_SIZES = [128, 16, 512, 32, 2048, 64, 256, 4]
TOY_TB = [1e-4, 2e-5, 3e-4, 1e-5, 5e-5, 1e-5, 2e-4, 1e-5]


_MODELS = ['resnet20', 'resnet50', 'densenet201', 'vgg16i', 'lstm']
_WORLDS = [(2, '10GbE'), (4, '10GbE'), (8, '10GbE'), (8, '56GbIB'), (16, '56GbIB')]
_THRESHOLDS = [0, 1000, 65536, 1 << 20, 524288000]
_MG_CASES = [(d, w, c) for d in _MODELS for (w, c) in _WORLDS]
_layers_cache = {}


def _model_layers(dnn):
    if dnn not in _layers_cache:
        from mgwfbp_b200.models import create_net
        kw = dict(vocab_size=10000, batch_size=20) if dnn == 'lstm' else {}
        with torch.device('meta'):
            net, _ = create_net(1000 if dnn not in ('resnet20', 'lstm') else 10, dnn, **kw)
        _layers_cache[dnn] = [[n, p.numel()] for n, p in net.named_parameters()]
    return _layers_cache[dnn]


def _synthetic_tb(dnn, world):
    layers = _model_layers(dnn)
    rng = np.random.RandomState(len(layers) * 7 + world)
    total = {'resnet20': 8e-3, 'resnet50': 60e-3, 'densenet201': 90e-3, 'vgg16i': 120e-3, 'lstm': 50e-3}[dnn]
    w = rng.rand(len(layers)) + 0.05
    return list((w / w.sum() * total).astype(float))


@pytest.fixture(scope='module')
def oracle_answers(reference_dir):
    """All reference-oracle questions of this module, answered by ONE subprocess."""
    reqs, keys = [], []

    def ask(key, layers, world, connection='10GbE', adaptive=True, tb=None, threshold=0, run_backward=False):
        keys.append(key)
        reqs.append(dict(reference_dir=reference_dir, world=world, connection=connection, adaptive=adaptive,
                         threshold=threshold, layers=layers, tb=tb, run_backward=run_backward))
    for dnn in _MODELS:
        for world, conn in _WORLDS:
            if (dnn, world, conn) not in _MG_CASES:
                continue
            ask(('mg', dnn, world, conn), _model_layers(dnn), world, conn, True, _synthetic_tb(dnn, world))
    for thr in _THRESHOLDS:
        ask(('thr', thr), _model_layers('resnet50'), 4, adaptive=False, threshold=thr)
    ask(('calls',), [[n, s] for n, s in zip(TOY_NAMES, TOY_SIZES)], 4, '10GbE', True, TOY_TB, 0, True)
    env = dict(os.environ, PYTHONPATH='')
    res = subprocess.run([sys.executable, os.path.join(HERE, 'reference_oracle.py')], input=json.dumps(reqs),
                         capture_output=True, text=True, cwd='/tmp', env=env, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    answers = json.loads(res.stdout[res.stdout.index('['):])
    return dict(zip(keys, answers))


def test_toy_golden_mgwfbp_4_workers():
    ab = AlphaBeta(*TABLE_10GBE[4])
    s = groups_mgwfbp(TOY_NAMES, TOY_SIZES, TOY_TB, ab)
    assert s.groups == [['3.bias'], ['3.weight', '2.bias'], ['2.weight', '1.bias'], ['1.weight', '0.bias'], ['0.weight']]
    assert dict(zip(s.keys, s.offsets))['3.weight:2.bias'] == [0, 256]
    assert dict(zip(s.keys, s.offsets))['2.weight:1.bias'] == [0, 2048]
    assert dict(zip(s.keys, s.offsets))['1.weight:0.bias'] == [0, 512]
    assert s.group_sizes == [4, 320, 2080, 528, 128]


def test_toy_golden_mgwfbp_8_workers_single_group():
    s = groups_mgwfbp(TOY_NAMES, TOY_SIZES, TOY_TB, AlphaBeta(*TABLE_10GBE[8]))
    assert s.groups == [TOY_NAMES[::-1]]


@pytest.mark.parametrize('threshold,expected', [
    (0, [[n] for n in TOY_NAMES[::-1]]),
    (600, [['3.bias', '3.weight', '2.bias', '2.weight'], ['1.bias', '1.weight', '0.bias', '0.weight']]),
    (2200, [['3.bias', '3.weight', '2.bias', '2.weight'], ['1.bias', '1.weight', '0.bias', '0.weight']]),
    (524288000, [TOY_NAMES[::-1]]),
])
def test_toy_golden_threshold(threshold, expected):
    assert groups_by_threshold(TOY_NAMES, TOY_SIZES, threshold).groups == expected


def test_duplicate_names_rejected():
    assert not check_unique(['a', 'a'])
    with pytest.raises(ValueError):
        groups_mgwfbp(['a', 'a'], [1, 1], [1e-3, 1e-3], AlphaBeta(1e-5, 1e-9))


def test_digest_depends_on_grouping():
    a = groups_by_threshold(TOY_NAMES, TOY_SIZES, 0)
    b = groups_by_threshold(TOY_NAMES, TOY_SIZES, 600)
    assert a.digest() != b.digest()
    assert a.digest() == groups_by_threshold(TOY_NAMES, TOY_SIZES, 0).digest()


@pytest.mark.parametrize('dnn,world,connection', _MG_CASES)
def test_mgwfbp_matches_reference(oracle_answers, dnn, world, connection):
    layers = _model_layers(dnn)
    tb = _synthetic_tb(dnn, world)
    want = oracle_answers[('mg', dnn, world, connection)]
    table = TABLE_10GBE if connection == '10GbE' else TABLE_56GBIB
    got = groups_mgwfbp([n for n, _ in layers], [s for _, s in layers], tb, AlphaBeta(*table[world]))
    assert got.groups == want['groups']
    assert got.key_groupidx == want['key_groupidx']
    assert dict(zip(got.keys, got.offsets)) == want['offsets']


@pytest.mark.parametrize('threshold', _THRESHOLDS)
def test_threshold_matches_reference(oracle_answers, threshold):
    layers = _model_layers('resnet50')
    want = oracle_answers[('thr', threshold)]
    got = groups_by_threshold([n for n, _ in layers], [s for _, s in layers], threshold)
    assert got.groups == want['groups']
    assert got.key_groupidx == want['key_groupidx']
    assert dict(zip(got.keys, got.offsets)) == want['offsets']


def test_reference_allreduce_call_sequence(oracle_answers):
    assert oracle_answers[('calls',)]['calls'] == [['3.bias', 4], ['3.weight:2.bias', 320], ['2.weight:1.bias', 2080],
                                                   ['1.weight:0.bias', 528], ['0.weight', 128]]


def test_fit_alpha_beta_matches_sklearn():
    from sklearn.linear_model import LinearRegression
    rng = np.random.RandomState(0)
    sizes = np.array([8192 * i for i in range(1, 64)], dtype=np.float64)
    times = 3e-5 + 2e-10 * sizes * 4 + rng.randn(sizes.size) * 1e-7
    ab = fit_alpha_beta(sizes, times)
    m = LinearRegression().fit((sizes * 4).reshape(-1, 1), times)
    assert ab.alpha == pytest.approx(m.intercept_, rel=1e-9, abs=1e-15)
    assert ab.beta == pytest.approx(m.coef_[0], rel=1e-9)


def test_table_lookup_any_world_size():
    assert table_lookup('10GbE', 8) == AlphaBeta(*TABLE_10GBE[8], name='10GbE')
    ab3 = table_lookup('10GbE', 3)
    assert TABLE_10GBE[2][0] < ab3.alpha < TABLE_10GBE[4][0]
    assert table_lookup('56GbIB', 32).alpha > TABLE_56GBIB[16][0]
    assert table_lookup('10GbE', 1)(1024) == 0.0


def test_piecewise_model_picks_cheapest_algorithm():
    pw = PiecewiseAlphaBeta(((0, 1 << 20, AlphaBeta(5e-6, 1e-9, 'oneshot')), (0, float('inf'), AlphaBeta(1.2e-5, 2e-12, 'twoshot'))))
    assert pw.choose(1024) == 'oneshot'
    assert pw.choose(1 << 24) == 'twoshot'
    assert pw(0) == 0.0
    assert pw.startup(1024) == 5e-6
    fitted = fit_piecewise({'a': ([1, 2, 3], [1.0, 2.0, 3.0])})
    assert fitted.pieces[0][2].beta == pytest.approx(0.25)


def test_simulation_orders_policies_sensibly():
    ab = AlphaBeta(*TABLE_10GBE[4])
    mg = groups_mgwfbp(TOY_NAMES, TOY_SIZES, TOY_TB, ab)
    wf = groups_by_threshold(TOY_NAMES, TOY_SIZES, 0)
    sim_mg = simulate_schedule(mg, TOY_NAMES, TOY_SIZES, TOY_TB, ab)
    sim_wf = simulate_schedule(wf, TOY_NAMES, TOY_SIZES, TOY_TB, ab)
    assert sim_mg['finish'] <= sim_wf['finish'] + 1e-12
    assert sim_mg['finish'] == pytest.approx(mg.predicted['tb_plus_tc'])


# ----------------------------------------------------------------------------- interference-aware selection
def _random_model(seed, L=60):
    rng = np.random.RandomState(seed)
    names = ['layer%d' % i for i in range(L)]
    sizes = [int(rng.choice([64, 256, 2048, 36864, 147456, 589824, 2359296])) for _ in range(L)]
    tb = [float(t) for t in rng.uniform(5e-6, 120e-6, L)]
    return names, sizes, tb


@pytest.mark.parametrize('seed', [0, 1, 2])
def test_contended_selection_with_zero_interference_is_plain_mgwfbp(seed):
    from mgwfbp_b200.parallel.scheduler import groups_mgwfbp_contended, simulate_contended
    names, sizes, tb = _random_model(seed)
    cost = AlphaBeta(12e-6, 3e-12)
    plain = groups_mgwfbp(names, sizes, tb, cost)
    assert groups_mgwfbp_contended(names, sizes, tb, cost, 0.0).groups == plain.groups
    # without interference the contended timeline is the ordinary one
    a = simulate_contended(plain, names, sizes, tb, cost, 0.0)
    b = simulate_schedule(plain, names, sizes, tb, cost)
    assert a['finish'] == pytest.approx(b['finish'], rel=1e-12)
    assert a['backward_end'] == pytest.approx(sum(tb), rel=1e-12)


@pytest.mark.parametrize('seed', [0, 1, 2])
def test_full_interference_makes_every_message_cost_its_time_and_selects_one_group(seed):
    from mgwfbp_b200.parallel.scheduler import groups_mgwfbp_contended, simulate_contended
    names, sizes, tb = _random_model(seed)
    cost = AlphaBeta(12e-6, 3e-12)
    for sched in (groups_by_threshold(names, sizes, 0), groups_by_threshold(names, sizes, 1 << 20), groups_mgwfbp(names, sizes, tb, cost)):
        sim = simulate_contended(sched, names, sizes, tb, cost, 1.0)
        assert sim['finish'] == pytest.approx(sum(tb) + sim['merged_tc_sum'], rel=1e-9)
    chosen = groups_mgwfbp_contended(names, sizes, tb, cost, 1.0)
    assert len(chosen.groups) == 1 and sorted(chosen.groups[0]) == sorted(names)
    assert chosen.predicted['contended_finish'] == pytest.approx(sum(tb) + cost(4 * sum(sizes)), rel=1e-9)
    # every candidate that was looked at is listed, and the winner is the minimum
    assert min(f for _, _, f in chosen.predicted['candidates']) == pytest.approx(chosen.predicted['contended_finish'])


def test_contended_finish_grows_with_interference_and_partial_interference_keeps_some_overlap():
    from mgwfbp_b200.parallel.scheduler import groups_mgwfbp_contended, simulate_contended
    names, sizes, tb = _random_model(3, L=120)
    cost = AlphaBeta(15e-6, 4e-12)
    sched = groups_by_threshold(names, sizes, 1 << 21)
    finishes = [simulate_contended(sched, names, sizes, tb, cost, r)['finish'] for r in (0.0, 0.25, 0.5, 0.75, 1.0)]
    assert all(b >= a - 1e-15 for a, b in zip(finishes, finishes[1:]))
    mid = groups_mgwfbp_contended(names, sizes, tb, cost, 0.25)
    n_plain = len(groups_mgwfbp(names, sizes, tb, cost).groups)
    assert 1 < len(mid.groups) < n_plain          # between the latency-only schedule and a single message
    assert mid.predicted['interference'] == 0.25
    # the chosen schedule is a valid partition in backward order
    flat = [n for g in mid.groups for n in g]
    assert flat == list(reversed(names))
    assert mid.group_sizes == [sum(sizes[names.index(n)] for n in g) for g in mid.groups]


def test_time_sliced_groups_cover_everything_in_backward_order():
    from mgwfbp_b200.parallel.scheduler import groups_time_sliced
    names = ['l%d' % i for i in range(12)]
    sizes = [100, 200, 300, 1000, 5000, 20000, 30000, 40000, 100000, 2000, 7, 50000]
    tb = [1, 1, 2, 2, 3, 3, 4, 4, 5, 1, 1, 3]
    for k in (1, 2, 3, 5, 40):
        s = groups_time_sliced(names, sizes, tb, k, tail_elems=700)
        flat = [n for g in s.groups for n in g]
        assert flat == list(reversed(names))                       # every tensor once, last layer first
        assert s.groups[-1] == ['l2', 'l1', 'l0']                  # the tail: trailing tensors up to 700 elements
        assert 2 <= len(s.groups) <= min(k, 9) + 1 and (k > 3 or len(s.groups) == k + 1)
        assert s.group_sizes == [sum(sizes[int(n[1:])] for n in g) for g in s.groups]
        assert all(s.key_groupidx[n] == gi for gi, g in enumerate(s.groups) for n in g)
    # equal slices of backward time: 30 units over the nine head tensors, three slices of about 10
    s = groups_time_sliced(names, sizes, tb, 3, tail_elems=700)
    spans = [sum(tb[int(n[1:])] for n in g) for g in s.groups[:-1]]
    assert spans == [10, 11, 5] or max(spans) <= 12
    # a tail budget smaller than the first tensor still leaves that tensor in the last group
    assert groups_time_sliced(names, sizes, tb, 2, tail_elems=1).groups[-1] == ['l0']


def test_late_groups_are_those_ready_close_to_the_end_of_backward():
    """``late_full``: a group counts as late when less than settings.LATE_GROUP_MS of profiled backward time is left once its
    earliest layer is done; the schedule's last group never does (it has the GPU to itself anyway)."""
    import torch
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.parallel.scheduler import groups_by_threshold
    net = torch.nn.Sequential(*[torch.nn.Linear(8, 8) for _ in range(6)])
    names = [n for n, _ in net.named_parameters()]
    times = [1e-4] * len(names)                     # 0.1 ms of backward per tensor
    schedule = lambda n, s, t: groups_by_threshold(n, s, 150)           # groups of 5, 5 and 2 tensors, last to first

    def build(**kw):
        return hvd.DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=0.1), named_parameters=net.named_parameters(),
                                        seq_layernames=names, layerwise_times=times, schedule=schedule, **kw)
    assert settings.LATE_GROUP_MS == pytest.approx(0.4)
    assert sorted(build()._late_groups) == []
    opt = build(late_full=True)
    assert [len(g) for g in opt._groups] == [5, 5, 2]
    # group 1 ends with '1.weight': two tensors (0.2 ms) are left after it -> late; group 0 leaves 0.7 ms -> not late
    assert sorted(opt._late_groups) == [1]
