# -*- coding: utf-8 -*-
"""Drop-in module for scripts that do ``import settings``; the switches live in the package."""
import sys as _sys
import mgwfbp_b200.settings as _impl

# Alias (not copy) so that ``settings.ADAPTIVE_MERGE = False`` edits the switch the package reads.
_sys.modules[__name__] = _impl
