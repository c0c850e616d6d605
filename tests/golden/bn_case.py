"""The small BatchNorm model shared by the golden generator (unmodified reference) and the tests (this front end):
layer list, seeded initial weights and data."""
import numpy as np

# SGD, not Adam: Adam divides every gradient entry by its own magnitude, so entries near zero (there are some behind the
# normalisation layers) turn rounding differences between engines into steps of size lr.
N, CLASSES, STEPS, LR, MOMENTUM = 12, 5, 2, 5e-2, 0.9


def layers(S):
    return [S.Input((1, 8, 8)), S.Conv2D(4, 1, (3, 3), "relu", stride=1, zero_padding=1), S.BatchNorm2d(4),
            S.MaxPool2D((2, 2), stride=2), S.Flatten(), S.Dense(64, 16, activation="relu"), S.BatchNorm1d(16),
            S.Dense(16, CLASSES, activation="softmax")]


def weights():
    rs = np.random.RandomState(77)
    f = lambda *s: (rs.standard_normal(s) * 0.3).astype(np.float32)
    return {1: (f(4, 1, 3, 3), f(1, 4, 1, 1)), 2: (1 + f(4), f(4)), 5: (f(64, 16), f(1, 16)), 6: (1 + f(16), f(16)),
            7: (f(16, CLASSES), f(1, CLASSES))}


def data():
    rs = np.random.RandomState(78)
    X = rs.standard_normal((N, 1, 8, 8)).astype(np.float32)
    Y = np.eye(CLASSES, dtype=np.float32)[rs.randint(0, CLASSES, N)]
    return X, Y
