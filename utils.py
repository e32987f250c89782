# -*- coding: utf-8 -*-
"""Drop-in module for ``import utils``."""
from mgwfbp_b200.utils.misc import *  # noqa: F401,F403
from mgwfbp_b200.utils.misc import s, predict_allreduce_time_with_size  # noqa: F401
