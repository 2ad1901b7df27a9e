"""Test-side alias of the package's seeded synthetic inputs (configurations, logits, activations, constructed blocks)."""
from project_maya_b200.synthetic import *  # noqa: F401,F403
from project_maya_b200.synthetic import BLOCK, CONFIGS, INF  # noqa: F401
