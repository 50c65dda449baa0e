"""``import pytensorpipe as tp`` keeps working: the names of the reference's Python module
(tensorpipe/python/tensorpipe.cc) served by tensorpipe_b200."""
from tensorpipe_b200.pytensorpipe import *  # noqa: F401,F403
from tensorpipe_b200.pytensorpipe import __all__  # noqa: F401
