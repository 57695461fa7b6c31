"""The parity protocol lives beside the oracle (oracle/parity.py) so that the bench's in-run check
can use the same functions; the tests import it under this name."""
from oracle.parity import *  # noqa: F401,F403
from oracle.parity import REPORT, REL  # noqa: F401
