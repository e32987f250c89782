# -*- coding: utf-8 -*-
"""``import models.lstm as lstmpy`` compatibility."""
from mgwfbp_b200.models.lstm import lstm, repackage_hidden  # noqa: F401
