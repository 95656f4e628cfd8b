"""IntentIR graphs of the benchmark configurations, as the reference's deterministic builders
emit them (``pipeline/tilelang/core.py``: ``any_kernel_dim`` :115-130, ``group_norm_kernel``
:175-242, ``softmax_inner`` :259-274, ``rms_norm2d`` :735-776, ``matmul_bias_relu2d`` :886-910,
``masked_softmax2d`` :1050-1076, ``layer_norm_persistent`` :1322-1384, ``layer_norm_residual2d``
:1426, ``add_bias2d``), stored in the JSON wire format of ``IntentFunction.to_json_dict``
(intent_ir/ir/ir_types.py:273-291).  ``tests/golden/make_golden.py`` writes the file from the
reference; the benchmark and the smoke entry read the graphs from here.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config_graphs.json")
_CACHE: Dict[str, Any] = {}


def config_graphs() -> Dict[str, Dict[str, Any]]:
    """name -> graph JSON (a fresh deep copy each call: callers edit dtypes in place)."""
    if not _CACHE:
        with open(_PATH) as f:
            _CACHE.update(json.load(f))
    return json.loads(json.dumps(_CACHE))


def config_graph(name: str) -> Dict[str, Any]:
    graphs = config_graphs()
    if name not in graphs:
        raise KeyError(f"no benchmark graph named {name!r}; have {sorted(graphs)}")
    return graphs[name]
