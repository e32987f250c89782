"""Import stub: the reference imports SummaryWriter but never constructs one (``dist_trainer.py:19,137``)."""


class SummaryWriter(object):
    def __init__(self, *a, **k):
        pass

    def add_scalar(self, *a, **k):
        pass

    def add_histogram(self, *a, **k):
        pass

    def close(self):
        pass
