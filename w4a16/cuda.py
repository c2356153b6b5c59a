from nibble_b200.cuda import *  # noqa: F401,F403
from nibble_b200 import cuda as _impl

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
