"""The CPU oracle's ctypes binding lives beside the oracle; tests import it through this name."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "oracle"))
from df_oracle_binding import *  # noqa: F401,F403,E402
from df_oracle_binding import lib  # noqa: F401,E402
