"""Process-wide logger, quiet by default.

The reference logs through one stdlib logger at WARNING with INFO lines for the
backend, the weight table and the missing/unexpected keys
(src/torchlet/logger.py:12-32, v10_triton_paged_gqa/llm.py:28-54).  Same here;
``TORCHLET_B200_LOG=INFO`` raises the level.
"""
from __future__ import annotations

import logging
import os
import sys

_FORMAT = "%(levelname).1s %(asctime)s %(name)s (%(module)s:%(lineno)d) %(message)s"


def get_logger(name: str = "torchlet_b200") -> logging.Logger:
    log = logging.getLogger(name)
    if not log.handlers:
        handler = logging.StreamHandler(sys.stderr)
        handler.setFormatter(logging.Formatter(_FORMAT, datefmt="%H:%M:%S"))
        log.addHandler(handler)
        log.propagate = False
        level = os.environ.get("TORCHLET_B200_LOG", "WARNING").upper()
        log.setLevel(getattr(logging, level, logging.WARNING))
    return log


logger = get_logger()
