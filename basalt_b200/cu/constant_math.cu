// Everything here is known at compile time: the stored value folds to one constant and the
// unread temporary disappears.
#define BASE (2 + 3)
__global__ void constant_math(int *out) {
    int a = BASE;
    int b = a * 4;
    int never_read = a + b;
    out[0] = b;
}
