// Empty stand-in: the reference includes <numa.h> in src/main.cu only and calls nothing from it.
