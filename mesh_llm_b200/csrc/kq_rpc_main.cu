// b200-rpc-server: the process mesh-llm spawns as a worker stage,
//   rpc-server -d <devices> -H <host> -p <port> --gguf <model.gguf>
// (mesh-llm/src/inference/launch.rs:887-933), backed by this library.  Unknown options that take a
// value in the reference's server (-c cache directory, -t threads, -m memory) are accepted and ignored.
#include "../../include/b200_kquant.h"

#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

static volatile sig_atomic_t g_stop = 0;
static void on_signal(int) { g_stop = 1; }

int main(int argc, char **argv) {
    const char *host = "127.0.0.1", *gguf = nullptr, *devices = nullptr;
    int port = 50052;
    for (int i = 1; i < argc; i++) {
        const char *a = argv[i];
        auto value = [&]() -> const char * {
            if (i + 1 >= argc) {
                fprintf(stderr, "%s needs a value\n", a);
                exit(2);
            }
            return argv[++i];
        };
        if (!strcmp(a, "-H") || !strcmp(a, "--host")) host = value();
        else if (!strcmp(a, "-p") || !strcmp(a, "--port")) port = atoi(value());
        else if (!strcmp(a, "-d") || !strcmp(a, "--device")) devices = value();
        else if (!strcmp(a, "--gguf")) gguf = value();
        else if (!strcmp(a, "-c") || !strcmp(a, "--cache") || !strcmp(a, "-t") || !strcmp(a, "--threads") ||
                 !strcmp(a, "-m") || !strcmp(a, "--mem")) value();
        else if (!strcmp(a, "-h") || !strcmp(a, "--help")) {
            printf("usage: %s [-H host] [-p port] [-d B200_0,...] [--gguf model.gguf]\n", argv[0]);
            return 0;
        } else {
            fprintf(stderr, "unknown option %s\n", a);
            return 2;
        }
    }
    const int n_dev = b200_reg_device_count();
    if (n_dev <= 0) {
        fprintf(stderr, "no B200 device: %s\n", b200_last_error());
        return 1;
    }
    if (devices) {
        // device names come from b200_dev_name ("B200_<i>"); every listed name must exist
        char *list = strdup(devices);
        for (char *tok = strtok(list, ","); tok; tok = strtok(nullptr, ",")) {
            bool found = false;
            for (int d = 0; d < n_dev && !found; d++) {
                char name[32];
                found = b200_dev_name(d, name, sizeof(name)) == B200_OK && !strcmp(name, tok);
            }
            if (!found) {
                fprintf(stderr, "unknown device %s\n", tok);
                return 2;
            }
        }
        free(list);
    }
    b200_rpc_server *srv = nullptr;
    if (b200_rpc_server_start(host, port, gguf, &srv) != B200_OK) {
        fprintf(stderr, "cannot start: %s\n", b200_last_error());
        return 1;
    }
    signal(SIGINT, on_signal);
    signal(SIGTERM, on_signal);
    printf("b200-rpc-server: %d device(s), listening on %s:%d%s%s\n", n_dev, host, b200_rpc_server_port(srv),
           gguf ? ", local GGUF " : "", gguf ? gguf : "");
    fflush(stdout);
    while (!g_stop) usleep(100000);
    b200_rpc_server_stop(srv);
    return 0;
}
