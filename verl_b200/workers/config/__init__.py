from .actor import *  # noqa: F401,F403
from .checkpoint import *  # noqa: F401,F403
from .engine import *  # noqa: F401,F403
from .model import *  # noqa: F401,F403
from .optimizer import *  # noqa: F401,F403
from .rollout import *  # noqa: F401,F403
