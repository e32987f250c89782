# -*- coding: utf-8 -*-
"""Drop-in package for ``import models``: re-exports the model zoo of ``mgwfbp_b200.models``."""
from mgwfbp_b200.models import *  # noqa: F401,F403
from mgwfbp_b200.models import lstm as _lstm_ctor, repackage_hidden, create_net, LSTMAN4  # noqa: F401
from mgwfbp_b200.models import lstm as lstm_module  # noqa: F401
