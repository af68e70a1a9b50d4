"""Package logger (counterpart of omni_npu/logger.py:18-58: one named logger
with a compact formatter; when vLLM is present its dictConfig is extended
instead of replaced)."""
from __future__ import annotations

import logging
import os

_FORMAT = "%(levelname)s %(asctime)s [%(name)s %(filename)s:%(lineno)d] %(message)s"

logger = logging.getLogger("omni_npu_b200")


def configure(level: str | None = None) -> logging.Logger:
    level = (level or os.environ.get("OMNI_B200_LOG_LEVEL", "INFO")).upper()
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
        logger.addHandler(h)
        logger.propagate = False
    logger.setLevel(level)
    return logger


def update_vllm_logging_config() -> None:
    """Add this package's logger to vLLM's logging configuration if vLLM is importable."""
    try:
        from vllm.logger import DEFAULT_LOGGING_CONFIG  # type: ignore
    except Exception:
        configure()
        return
    cfg = DEFAULT_LOGGING_CONFIG
    cfg.setdefault("formatters", {})["omni_b200"] = {"format": _FORMAT, "datefmt": "%m-%d %H:%M:%S"}
    cfg.setdefault("handlers", {})["omni_b200"] = {"class": "logging.StreamHandler",
                                                   "formatter": "omni_b200", "level": "INFO",
                                                   "stream": "ext://sys.stdout"}
    cfg.setdefault("loggers", {})["omni_npu_b200"] = {"handlers": ["omni_b200"], "level": "INFO",
                                                      "propagate": False}
    configure()


configure()
