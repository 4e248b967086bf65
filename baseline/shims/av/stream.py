class Stream:  # type annotation only
    pass
