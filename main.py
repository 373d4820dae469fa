"""Launch command of the serving engine: ``python main.py --model DIR --host H --port P``."""

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from b200serve.api.server import main  # noqa: E402

if __name__ == "__main__":
    main()
