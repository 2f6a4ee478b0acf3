"""``import muon`` compatibility module: the reference is distributed as a single module
named ``muon``; this one re-exports the same public names from ``muon_b200``."""
from muon_b200 import *  # noqa: F401,F403
from muon_b200 import __all__  # noqa: F401
