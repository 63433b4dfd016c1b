class ActorHandle:
    pass
