"""``matplotlib.pyplot`` whose every function accepts anything and draws nothing."""


def __getattr__(name):
    def nothing(*args, **kwargs):
        return None
    return nothing
