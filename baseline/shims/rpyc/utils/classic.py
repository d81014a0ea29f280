def obtain(x):
    return x
