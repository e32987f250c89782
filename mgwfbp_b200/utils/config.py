# -*- coding: utf-8 -*-
"""Reader for ``exp_configs/<dnn>.conf``.

The files are bash fragments (``key=value`` and ``key="${key:-default}"`` /
``: "${key:=default}"``) that the launch scripts ``source``; this parser lets Python entry
points and tests read the same files without a shell.  Environment variables override
``${var:-default}`` forms exactly as bash would.
"""
from __future__ import annotations

import os
import re
from typing import Dict, Mapping, Optional

_ASSIGN = re.compile(r'^\s*([A-Za-z_][A-Za-z0-9_]*)=(.*)$')
_COLON_DEFAULT = re.compile(r'^\s*:\s*"?\$\{([A-Za-z_][A-Za-z0-9_]*):=([^}]*)\}"?\s*$')
_PARAM = re.compile(r'\$\{([A-Za-z_][A-Za-z0-9_]*)(?::-([^}]*))?\}')

CONFIG_KEYS = ('lr', 'batch_size', 'dnn', 'dataset', 'max_epochs', 'nstepsupdate', 'data_dir')


def _expand(value: str, env: Mapping[str, str], scope: Mapping[str, str]) -> str:
    def repl(m):
        name, default = m.group(1), m.group(2)
        cur = scope.get(name, env.get(name))
        if cur:
            return cur
        return default if default is not None else ''
    return _PARAM.sub(repl, value)


def parse_conf(path: str, env: Optional[Mapping[str, str]] = None) -> Dict[str, str]:
    env = os.environ if env is None else env
    out: Dict[str, str] = {}
    with open(path) as f:
        for raw in f:
            line = raw.split('#', 1)[0].strip() if not raw.lstrip().startswith('#') else ''
            if not line:
                continue
            m = _COLON_DEFAULT.match(line)
            if m:
                name, default = m.group(1), m.group(2)
                cur = out.get(name, env.get(name))
                out[name] = cur if cur else _expand(default, env, out)
                continue
            m = _ASSIGN.match(line)
            if not m:
                continue
            name, value = m.group(1), m.group(2).strip()
            if len(value) >= 2 and value[0] == value[-1] and value[0] in '"\'':
                value = value[1:-1]
            out[name] = _expand(value, env, out)
    return out


def load_experiment(dnn: str, config_dir: Optional[str] = None, env: Optional[Mapping[str, str]] = None) -> Dict[str, object]:
    """Typed view of one experiment file."""
    if config_dir is None:
        config_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), 'exp_configs')
    raw = parse_conf(os.path.join(config_dir, dnn + '.conf'), env)
    typed: Dict[str, object] = dict(raw)
    for k, cast in (('lr', float), ('batch_size', int), ('max_epochs', int), ('nstepsupdate', int)):
        if k in raw and raw[k] != '':
            typed[k] = cast(raw[k])
    return typed
