"""Where the reference tree is: the REF environment variable, else a directory named `reference` beside
this repository.  None when neither exists (the checker then relies on the committed fixtures only)."""
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def find():
    cands = [os.environ.get("REF"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "kvcomp_cuda_extension")):
            return c
    return None


def require():
    root = find()
    if root is None:
        raise FileNotFoundError("reference tree not found: set REF to its root")
    return root
