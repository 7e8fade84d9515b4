"""Import name of the engine.

The source tree lives in the folder ``llm-serving-engine_b200`` next to this one. A hyphen cannot
appear in a Python module name, so this package only points its search path at that folder: every
``llmserve_b200.<sub>`` import resolves to ``llm-serving-engine_b200/<sub>``.
"""

from pathlib import Path as _Path

__path__ = [str(_Path(__file__).resolve().parent.parent / "llm-serving-engine_b200")]

from ._exports import *  # noqa: E402,F401,F403
from ._exports import __all__  # noqa: E402,F401
