"""railgun_b200: a small inference engine for one B200, after Atari-Katana/railgun."""
import logging
import os

__version__ = "0.2.0"

log = logging.getLogger("railgun_b200")
_LEVELS = {"error": logging.ERROR, "warn": logging.WARNING, "warning": logging.WARNING, "info": logging.INFO,
           "debug": logging.DEBUG, "trace": logging.DEBUG}


def init_logging(level: str | None = None) -> None:
    """Messages of the package go to standard error at the level ``RAILGUN_LOG`` names (error, warn, info, debug;
    default info), as the reference's command line filters its log by an environment variable with "info" as
    the default (crates/vllm-cli/src/main.rs:40-49).  Progress lines of native builds are info."""
    name = (level or os.environ.get("RAILGUN_LOG", "info")).lower()
    if not log.handlers:
        handler = logging.StreamHandler()
        handler.setFormatter(logging.Formatter("[railgun_b200] %(message)s"))
        log.addHandler(handler)
        log.propagate = False
    log.setLevel(_LEVELS.get(name, logging.INFO))


init_logging()
