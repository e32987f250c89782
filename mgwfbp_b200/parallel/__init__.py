# -*- coding: utf-8 -*-
"""Data-parallel machinery: runtime, merge scheduler, cost model, communicators, optimizer."""
