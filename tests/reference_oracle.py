"""Run the reference's unmodified grouping code as an oracle, in a separate process.

Reads a JSON list of requests on stdin, writes a JSON list of answers on stdout (one process
serves many requests because importing torch and the reference dominates the cost).  The reference file
``distributed_optimizer.py`` is imported from the reference checkout (never copied) with
``horovod.torch.mpi_ops`` replaced by an in-process stub that records all-reduce calls.

request: {"reference_dir", "world", "connection", "adaptive", "threshold", "layers": [[name, numel], ...],
          "tb": [...]|null, "run_backward": bool}
answer:  {"groups": [[names]], "key_groupidx": {...}, "offsets": {key: [..]}, "calls": [[name, numel], ...]}
"""
import collections
import collections.abc
import json
import sys
import types


def main():
    reqs = json.load(sys.stdin)
    ref = reqs[0]['reference_dir']
    state = {'world': reqs[0]['world']}
    # the reference is a flat directory of modules (settings, utils, profiling, ...): the repository under test has
    # modules of the same names at its root, so its directory (passed in the request) must not be importable here
    import os
    repo = os.path.abspath(reqs[0].get('repo_root') or os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path[:] = [ref] + [p for p in sys.path if p not in ('', ref) and os.path.abspath(p) != repo]
    collections.Iterable = collections.abc.Iterable
    calls = []
    ops = types.ModuleType('horovod.torch.mpi_ops')
    ops.size = lambda: state['world']
    ops.local_size = lambda: state['world']
    ops.rank = lambda: 0
    ops.local_rank = lambda: 0
    ops.init = lambda: None

    def allreduce_async_(tensor, average=True, name=None):
        calls.append([name, int(tensor.numel())])
        return tensor
    ops.allreduce_async_ = allreduce_async_
    ops.allgather_async = lambda t, name=None: t
    ops.broadcast_async_ = lambda t, root_rank, name=None: t
    ops.synchronize = lambda h: h
    ops.broadcast = lambda t, root_rank, name=None: t
    hv = types.ModuleType('horovod')
    hvt = types.ModuleType('horovod.torch')
    hv.torch, hvt.mpi_ops = hvt, ops
    sys.modules.update({'horovod': hv, 'horovod.torch': hvt, 'horovod.torch.mpi_ops': ops})

    import logging
    import torch
    import settings
    settings.logger.setLevel(logging.ERROR)
    import distributed_optimizer as ref_opt
    answers = []
    for req in reqs:
        del calls[:]
        state['world'] = req['world']
        settings.CONNECTION = req['connection']
        settings.ADAPTIVE_MERGE = bool(req['adaptive'])
        ref_opt.ADAPTIVE_MERGE = bool(req['adaptive'])
        params = collections.OrderedDict()
        for name, numel in req['layers']:
            # meta tensors carry sizes without memory; only the backward case needs real storage
            dev = 'cpu' if req.get('run_backward') else 'meta'
            params[name] = torch.nn.Parameter(torch.zeros(int(numel), device=dev))
        sgd = torch.optim.SGD(list(params.values()), lr=0.1)
        names = [n for n, _ in req['layers']]
        tb = req.get('tb')
        opt = ref_opt.DistributedOptimizer(sgd, named_parameters=list(params.items()),
                                           seq_layernames=names if tb is not None else None,
                                           layerwise_times=tb, threshold=req.get('threshold', 0))
        out = {'groups': opt._groups, 'key_groupidx': opt._key_groupidx_maps,
               'offsets': {k: list(map(int, v)) for k, v in opt._merged_parameter_offsets.items()}}
        if req.get('run_backward'):
            # a chain in which each parameter is used after the previous one, so that the
            # gradient accumulators fire last layer first
            h = torch.ones(1)
            for name in names:
                h = (h + params[name].sum()) * 1.0
            h.sum().backward()
            out['calls'] = [list(c) for c in calls]
        answers.append(out)
    json.dump(answers, sys.stdout)


if __name__ == '__main__':
    main()
