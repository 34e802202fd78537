import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, 'tests', 'golden')):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run with -m gpu on a B200)')


def pytest_sessionfinish(session, exitstatus):
    """Write the errors the comparisons observed (tests/util.py:OBSERVED) where NSA_PARITY_REPORT points."""
    path = os.environ.get('NSA_PARITY_REPORT')
    if not path:
        return
    import json
    import util
    if util.OBSERVED:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, 'w') as f:
            json.dump(util.OBSERVED, f, indent=1, sort_keys=True)
