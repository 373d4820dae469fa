"""Import alias for the engine package.

The sources live in ``qwen36-mi250-tracelab-20261107_b200/`` at the repository
root. That directory name is not a valid Python identifier, so this module
redirects its own search path there: ``import b200serve.models`` resolves to
``qwen36-mi250-tracelab-20261107_b200/models``.
"""

import os as _os

_ROOT = _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))
SOURCE_DIR = _os.path.join(_ROOT, "qwen36-mi250-tracelab-20261107_b200")
__path__ = [SOURCE_DIR]
__version__ = "0.1.0"
