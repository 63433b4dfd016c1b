class NodeAffinitySchedulingStrategy:
    def __init__(self, *args, **kwargs):
        pass
