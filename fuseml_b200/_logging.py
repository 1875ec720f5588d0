"""Package logger (``logging.getLogger("fuseml")``), same name as the reference's
(fuseml/_logging.py:7-12) so existing logging configuration keeps working."""
import logging

logger = logging.getLogger("fuseml")
if not logger.handlers and not logging.getLogger().handlers:
    logging.basicConfig(level=logging.WARNING, format="[%(name)s] %(levelname)s: %(message)s")
