def generate(ref, here): pass
