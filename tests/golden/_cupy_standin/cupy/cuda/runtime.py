def getDeviceCount():
    return 0


def deviceSynchronize():
    pass
