"""Per-module loggers (counterpart of python/brt/runtime/log.py in the reference)."""
import logging
import os

_LEVEL = os.environ.get("BRT_LOG_LEVEL", "WARNING").upper()


def get_logger(name: str = "brainstorm_b200") -> logging.Logger:
    logger = logging.getLogger(os.path.splitext(os.path.basename(name))[0] if os.sep in name
                               else name)
    if not logger.handlers:
        handler = logging.StreamHandler()
        handler.setFormatter(logging.Formatter("%(levelname)s %(name)s: %(message)s"))
        logger.addHandler(handler)
        logger.propagate = False
    logger.setLevel(getattr(logging, _LEVEL, logging.WARNING))
    return logger


def set_level(level: str) -> None:
    logging.getLogger("brainstorm_b200").setLevel(level.upper())
