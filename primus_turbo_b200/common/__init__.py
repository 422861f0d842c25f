from .logger import logger  # noqa: F401
