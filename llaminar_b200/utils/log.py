"""Rank-prefixed logging; level from LLAMINAR_LOG_LEVEL or -v (reference: src/v2/utils/Logger.h)."""
import logging
import os

from .env import debug_env

_configured = False


def get_logger(name: str = "llaminar") -> logging.Logger:
    global _configured
    if not _configured:
        level = str(debug_env().log_level).upper()
        rank = os.environ.get("RANK", "0")
        logging.basicConfig(level=getattr(logging, level, logging.INFO),
                            format=f"%(asctime)s [rank {rank}] %(levelname)s %(name)s: %(message)s", datefmt="%H:%M:%S")
        _configured = True
    return logging.getLogger(f"llaminar.{name}")
