"""The index-checking build of the kernels (``MGWFBP_CHECKED=1``): same numerics, no report on sound tables, and a
report instead of an access when a table is inconsistent.  The inconsistency is made on the host (an element count
lowered below what the offset table says), a state in which the normal build would merely leave the tail of that
tensor untouched, so neither build touches memory it should not."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = r'''
import ctypes as C, json, sys
import numpy as np
import torch
sys.path.insert(0, %(root)r)
from mgwfbp_b200.ops import _lib
from mgwfbp_b200.ops.tables import GroupTable, HyperTable
from mgwfbp_b200.parallel.comm.nvl import NvlComm
lib = _lib.load()
assert _lib.is_checked()
out = {}
torch.manual_seed(0)
dev = torch.device('cuda')
sizes = [5, 4096, 100003, 7]
params = [torch.randn(n, device=dev) for n in sizes]
ref = [p.clone() for p in params]
moms = [torch.zeros_like(p) for p in params]
grads = [torch.randn_like(p) for p in params]
table = GroupTable(params, [0] * len(params), moms, dev)
table.refresh_grads(grads)
hyper = HyperTable(dev)
hyper.sync([dict(lr=0.1, weight_decay=1e-4, momentum=0.9, dampening=0.0, nesterov=False)])
s = torch.cuda.current_stream().cuda_stream
_lib.check(lib.mgw_multi_tensor_sgd(C.byref(table.struct), hyper.data_ptr(), None, 1.0, 1, _lib.MODE_UPDATE, None, 8, s))
torch.cuda.synchronize()
want = [r - 0.1 * (g + 1e-4 * r) for r, g in zip(ref, grads)]
out['sgd_ok'] = all(torch.allclose(p, w, rtol=1e-5, atol=1e-6) for p, w in zip(params, want))
out['sgd_report'] = _lib.bounds_report()

comm = NvlComm.shared()
res = {}
for algo in ('oneshot', 'twoshot'):
    x = torch.randn(100003, device=dev); keep = x.clone()
    comm.synchronize(comm.allreduce_async_(x, algo=algo))
    torch.cuda.synchronize(); comm.check_status()
    res[algo] = bool(torch.equal(x, keep))
stamps = _lib.phase_times(1)[0]              # the two-shot launch above: pack, barrier, reduce, barrier, consume
out['phases_monotone'] = bool(stamps[0] > 0 and all(a <= b for a, b in zip(stamps, stamps[1:])))
out['allreduce_ok'] = res
out['allreduce_report'] = _lib.bounds_report()

# host-made inconsistency: tensor 2 now claims 1003 elements while the offset table still gives it 25001 slots
raw = table.tensors.cpu().numpy().copy()
rec = raw.view(np.dtype([('param', '<u8'), ('mom', '<u8'), ('numel', '<i4'), ('pg', '<i4')]))
rec['numel'][2] = 1003
table.tensors.copy_(torch.from_numpy(raw))
before = params[2].clone()
_lib.check(lib.mgw_multi_tensor_sgd(C.byref(table.struct), hyper.data_ptr(), None, 1.0, 0, _lib.MODE_UPDATE, None, 8, s))
torch.cuda.synchronize()
out['tail_untouched'] = bool(torch.equal(params[2][1004:], before[1004:]))
out['bad_report'] = _lib.bounds_report()
out['report_cleared'] = _lib.bounds_report()
print('RESULT ' + json.dumps(out))
'''


def test_checked_build_is_silent_on_sound_tables_and_reports_a_bad_one():
    import json
    env = dict(os.environ, MGWFBP_CHECKED='1')       # the checked library is built on first use if it is not there yet
    res = subprocess.run([sys.executable, '-c', _CHILD % {'root': ROOT}], env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith('RESULT ')][-1]
    out = json.loads(line[len('RESULT '):])
    assert out['sgd_ok'] and out['sgd_report'] == []
    assert out['allreduce_ok'] == {'oneshot': True, 'twoshot': True} and out['allreduce_report'] == []
    assert out['phases_monotone']
    assert out['tail_untouched']
    assert len(out['bad_report']) == 1 and out['bad_report'][0]['unit'] == 'multi_tensor_sgd'
    assert out['bad_report'][0]['code'] in (3, 4)
    assert out['report_cleared'] == []
