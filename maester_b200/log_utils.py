"""Process-wide logger (reference: maester/log_utils.py:4-17)."""
import logging
import os

logger = logging.getLogger("maester_b200")


def init_logger(level: int = logging.INFO) -> None:
    root = logging.getLogger()
    root.setLevel(level)
    if not any(isinstance(h, logging.StreamHandler) for h in root.handlers):
        handler = logging.StreamHandler()
        handler.setLevel(level)
        handler.setFormatter(logging.Formatter("[%(asctime)s %(levelname)s %(name)s] %(message)s"))
        root.addHandler(handler)
    logger.setLevel(level)
    # the kineto profiler is chatty below this level
    os.environ.setdefault("KINETO_LOG_LEVEL", "5")
