available = False
