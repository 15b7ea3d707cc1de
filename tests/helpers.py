"""Engine factories for the tests: the package's example programs (attentionengine_b200/examples.py)."""
from attentionengine_b200.examples import *  # noqa: F401,F403
from attentionengine_b200.examples import meta_tensor  # noqa: F401
