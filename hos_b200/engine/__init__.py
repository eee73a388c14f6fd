"""The step function, the generation loop and the entry points.  Engine and Runner pull in
torch and the kernels, so they are loaded at first use (the command line answers --help
and bad options without them)."""


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    if name == "Runner":
        from .runner import Runner
        return Runner
    raise AttributeError(name)
